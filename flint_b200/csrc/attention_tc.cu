// Prefill attention on the tcgen05 tensor cores, over the paged bfloat16 cache.
//
// One block per (tile of up to 128 consecutive query rows of one request, query head).  The keys
// of the request are walked in tiles of 64, always read from the cache pages (so a portion of a
// prompt sees the keys of earlier portions as well as its own):
//   S = Q K^T        tcgen05.mma, Q [128, hd] and K [64, hd] both K-major in shared memory, S in
//                    tensor memory (128 lanes = query rows, 64 columns = keys)
//   softmax          one thread per query row reads its row of S with tcgen05.ld, applies scale,
//                    the causal and window mask, keeps the running reference and sum in float32,
//                    and writes P = exp2(s - reference) as bfloat16 back into tensor memory, over the first
//                    half of the scores it came from (tcgen05.st, two probabilities to a column)
//   O += P V         tcgen05.mma with P as the A operand from tensor memory and V [64 keys, hd] as an
//                    MN-major B operand from shared memory; O stays in tensor memory over all key tiles
//                    of the block.  (P in shared memory cost a 16 KB store and a proxy fence per tile and
//                    made every tile's probabilities wait for the P V of the tile before.)
// The reference of a row is its running maximum, but it only moves when the maximum has grown by more
// than 8 (a factor of 256 in P; any reference gives the same softmax as long as the sum and O use the
// same one).  Only then does the row's warp rescale its rows of O in tensor memory (load, multiply,
// store), which after the first few tiles is rare; otherwise a tile costs a thread one read of its 64
// scores, 64 exponentials and the store of P.
// The steps of neighbouring key tiles overlap: S has two buffers in tensor memory, and the MMA thread
// issues S of tile i+1 before it waits for P of tile i, so the tensor core computes the next scores
// while the rows' threads are busy with the softmax.
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
#include "attention_kernels.cuh"

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
  long long wait_cycles;     // limit of every wait on an mbarrier
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

// 64 consecutive columns of this thread's lane, then the wait, in one statement: nothing that uses the
// values can be scheduled before the wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :: "r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 consecutive 32-bit columns of this thread's lane (here: 64 bfloat16 of a row of P, two to a column)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
// D += A B with A [128, 16] bfloat16 in tensor memory (lane = row, two elements of K to a column) and B in shared memory
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 2^x on the special-function unit (float32 in and out, about 2 ulp)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(THREADS, 2)      // two blocks per SM: registers are held to that
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];   // tiles need 1024-byte alignment (128-byte swizzle)
  __shared__ __align__(8) uint64_t bars[13];  // q, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, o_full
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  pdl_launch();
  if (*(volatile int*)p.error_flag) return;
  // Blocks start in the order of their index, heads fastest: all heads of the last tile first.  Later tiles see
  // more keys, so the long blocks start first and the short ones fill in behind them; the heads of a kv group
  // run side by side and share their keys in L2.
  const int* tile = p.tiles + 4 * (gridDim.y - 1 - blockIdx.y);
  const int row0 = tile[0], n_rows = tile[1], slot = tile[2], pos0 = tile[3];
  const int head = blockIdx.x;
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

  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {           // would corrupt the swizzle: refuse rather than compute garbage
    if (threadIdx.x == 0) atomicExch(p.error_flag, 2);
    return;
  }
  const uint32_t q_smem = base;                                       // chunks x [128 rows][128 B]
  const uint32_t kv_smem = q_smem + chunks * BQ * 128;                // per stage: K chunks, then V chunks
  const uint32_t kv_stage_bytes = 2u * chunks * BKV * 128;
  // Keys and values have rings of their own: a key tile is free as soon as its scores are computed, well
  // before the values of the same tile are, so the next keys are on their way while the softmax still runs
  const uint32_t bar_q = smem_u32(&bars[0]), bar_kfull0 = smem_u32(&bars[1]), bar_kempty0 = smem_u32(&bars[3]);
  const uint32_t bar_vfull0 = smem_u32(&bars[5]), bar_vempty0 = smem_u32(&bars[7]);
  const uint32_t bar_s0 = smem_u32(&bars[9]), bar_p = smem_u32(&bars[11]), bar_o = smem_u32(&bars[12]);
  const uint32_t tmem_cols = 256;             // two score buffers of 64 columns, then up to 128 of output
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_kfull0 + 8 * s, 1);
      mbar_init(bar_kempty0 + 8 * s, 1);
      mbar_init(bar_vfull0 + 8 * s, 1);
      mbar_init(bar_vempty0 + 8 * s, 1);
    }
    mbar_init(bar_s0, 1);
    mbar_init(bar_s0 + 8, 1);
    mbar_init(bar_p, BQ);       // every softmax row arrives itself
    mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 2 * BKV;   // scores of tile i at tmem_s + (i & 1) * BKV
  volatile int* ab = &abort_flag;

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- loads
    // The barriers and the tensor memory above need nothing from earlier kernels; the queries and the newest
    // keys and values come from the kernel before this one.
    pdl_wait();
    mbar_expect_tx(bar_q, chunks * BQ * 128);
    for (int c = 0; c < chunks; ++c) tma_load_2d(q_smem + c * BQ * 128, &map_q, head * hd + c * 64, row0, bar_q);
    const int* bt = p.block_table + (size_t)slot * p.max_pages;
    // one operand (keys or values) of tile i into its half of stage i % STAGES
    auto load_tile = [&](int i, bool values) -> bool {
      const int s = i % STAGES;
      if (!mbar_wait((values ? bar_vempty0 : bar_kempty0) + 8 * s, ((i / STAGES) & 1) ^ 1, ab, p.wait_cycles)) return false;
      const uint32_t bar = (values ? bar_vfull0 : bar_kfull0) + 8 * s;
      mbar_expect_tx(bar, kv_stage_bytes / 2);
      const uint32_t dst = kv_smem + s * kv_stage_bytes + (values ? chunks * BKV * 128 : 0);
      const int kv0 = (tile_lo + i) * BKV;
      for (int pc = 0; pc < pieces; ++pc) {
        const int key = kv0 + pc * piece;
        const int lp = key / P;
        int page = lp < p.max_pages ? bt[lp] : -1;
        if (page < 0) page = 0;   // never visible to these queries (masked): any finite page will do
        const int row = (page * p.nkv + kvh) * P + key % P;
        for (int c = 0; c < chunks; ++c)
          tma_load_2d(dst + c * BKV * 128 + pc * piece * 128, values ? &map_v : &map_k, c * 64, row, bar);
      }
      return true;
    };
    // in the order in which the stages come free: K_0, K_1, V_0, then K_{i+2} (after S_i) and V_{i+1} (after P V of i-1)
    bool ok = load_tile(0, false);
    if (ok && n_kv_tiles > 1) ok = load_tile(1, false);
    if (ok) ok = load_tile(0, true);
    for (int i = 0; ok && i < n_kv_tiles; ++i) {
      if (i + 2 < n_kv_tiles) ok = load_tile(i + 2, false);
      if (ok && i + 1 < n_kv_tiles) ok = load_tile(i + 1, true);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issue
    const uint32_t idesc_s = idesc_f16(BKV, 0), idesc_o = idesc_f16(hd, 1);
    bool ok = mbar_wait(bar_q, 0, ab, p.wait_cycles);
    // S_i = Q K_i^T into score buffer i & 1, as soon as the keys of tile i have landed
    auto issue_scores = [&](int i) -> bool {
      const int s = i % STAGES;
      if (!mbar_wait(bar_kfull0 + 8 * s, (i / STAGES) & 1, ab, p.wait_cycles)) return false;
      tc_fence_after();
      const uint32_t k_src = kv_smem + s * kv_stage_bytes;
      for (int k = 0; k < hd / 16; ++k) {
        const uint32_t off = (k >> 2) * 128 * 128 + (k & 3) * 32;          // Q: 128 rows per chunk
        const uint32_t koff = (k >> 2) * BKV * 128 + (k & 3) * 32;         // K: 64 rows per chunk
        umma_bf16(tmem_s + (i & 1) * BKV, smem_desc(q_smem + off), smem_desc(k_src + koff), idesc_s, k > 0 ? 1u : 0u);
      }
      umma_commit(bar_s0 + 8 * (i & 1));
      umma_commit(bar_kempty0 + 8 * s);          // the keys are free once these MMAs have read them
      return true;
    };
    if (ok) ok = issue_scores(0);
    for (int i = 0; i < n_kv_tiles && ok; ++i) {
      // the next tile's scores first: their buffer was last read for tile i-1, whose P has been handed over
      if (i + 1 < n_kv_tiles) ok = issue_scores(i + 1);
      if (!ok) break;
      ok = mbar_wait(bar_p, i & 1, ab, p.wait_cycles);         // P is in shared memory, S has been read, O is rescaled
      if (!ok) break;
      const int s = i % STAGES;
      ok = mbar_wait(bar_vfull0 + 8 * s, (i / STAGES) & 1, ab, p.wait_cycles);
      if (!ok) break;
      tc_fence_after();
      const uint32_t v_src = kv_smem + s * kv_stage_bytes + chunks * BKV * 128;
      for (int k = 0; k < BKV / 16; ++k) {      // O_tile = P V over the 64 keys
        // V [keys, hd] is MN-major for B: 16 keys down = 2048 bytes; 64-wide chunks of hd are BKV*128 apart
        const uint64_t vd = smem_desc_mn(v_src + k * 16 * 128, BKV * 128, 1024);
        umma_bf16_a_tmem(tmem_o, tmem_s + (i & 1) * BKV + k * 8, vd, idesc_o, (i > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(bar_o);
      umma_commit(bar_vempty0 + 8 * s);
    }
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- softmax rows
    const int q = warp & 3;
    const int r = q * 32 + lane;                    // row of the tile = TMEM lane
    const bool row_ok = r < n_rows;
    const int q_pos = pos0 + (row_ok ? r : n_rows - 1);
    const int first = p.window > 0 ? max(0, q_pos + 1 - p.window) : 0;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    constexpr float kRescaleStep = 8.0f;            // in log2 units
    float ref = -1e30f, l = 0.f;                    // reference of the exponentials, sum of P
    bool ok = true;
    for (int i = 0; i < n_kv_tiles && ok; ++i) {
      ok = mbar_wait(bar_s0 + 8 * (i & 1), (i >> 1) & 1, ab, p.wait_cycles);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = (tile_lo + i) * BKV;
      // only tiles that touch the diagonal or the window's edge need the mask (uniform in the block)
      const bool need_mask = (kv0 + BKV - 1 > pos0) || (p.window > 0 && kv0 < pos0 + n_rows - p.window);
      float sc[BKV];
      tmem_ld64(tmem_s + (i & 1) * BKV + lane_addr, sc);
      // keys a row does not see get a score of minus infinity (their probability is then exactly zero); one pass
      // on the few tiles that need it keeps the loops below in one form
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BKV; ++c) {
          const int kj = kv0 + c;
          if (!(kj <= q_pos && kj >= first)) sc[c] = -INFINITY;
        }
      }
      // the maximum of the raw scores (the scale is positive), in four strands so that the chain is short
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BKV; ++c) m4[c & 3] = fmaxf(m4[c & 3], sc[c]);
      const float mraw = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      const float mx = fmaxf(ref, mraw * p.scale_log2);
      // Every thread waits for every P V in turn, each before it arrives for the next one (a wait by parity cannot
      // tell a barrier that is two phases ahead from one that is in step).  P V of the previous tile only has to
      // be done before O is touched; otherwise the wait comes after this tile's probabilities are written, when
      // it has long been done.
      bool o_seen = i == 0;
      if (__any_sync(0xffffffffu, mx - ref > kRescaleStep)) {      // uniform in the warp: tcgen05.ld/st are
        const float alpha = ex2(ref - mx);                          // warp-wide; every row of the warp moves
        ref = mx;
        l *= alpha;
        if (i > 0) {
          ok = mbar_wait(bar_o, (i - 1) & 1, ab, p.wait_cycles);
          if (!ok) break;
          o_seen = true;
          tc_fence_after();
          for (int d0 = 0; d0 < hd; d0 += 16) {
            float v[16];
            tmem_ld16(tmem_o + lane_addr + d0, v);
#pragma unroll
            for (int d = 0; d < 16; ++d) v[d] *= alpha;
            tmem_st16(tmem_o + lane_addr + d0, v);
          }
          tmem_st_wait();
        }
      }
      // probabilities, as bf16 back into tensor memory over the first half of the scores they came from (two
      // to a column: the A operand of P V); the row's sum is kept in float32 from the unrounded probabilities
      // (four strands)
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_ref = -ref;
      uint32_t packed[BKV / 2];
#pragma unroll
      for (int c = 0; c < BKV; c += 2) {
        float pr[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          pr[e] = ex2(fmaf(sc[c + e], p.scale_log2, neg_ref));
        }
        const __nv_bfloat162 b = __floats2bfloat162_rn(pr[0], pr[1]);
        s4[c & 2] += pr[0];
        s4[(c & 2) + 1] += pr[1];
        packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&b);
      }
      tmem_st32(tmem_s + (i & 1) * BKV + lane_addr, packed);
      tmem_st_wait();
      if (!o_seen) {
        ok = mbar_wait(bar_o, (i - 1) & 1, ab, p.wait_cycles);
        if (!ok) break;
      }
      l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
      // hand P (and the rescaled O) to the tensor core (the barrier counts all 128 rows; no thread waits on
      // another here)
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok) ok = mbar_wait(bar_o, (n_kv_tiles - 1) & 1, ab, p.wait_cycles);
    if (ok) {
      tc_fence_after();
      pdl_wait();             // every thread that writes waits for the earlier kernels itself (long over by now)
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(row0 + r) * p.nq + head) * hd;
      for (int d0 = 0; d0 < hd; d0 += 16) {           // the loads are warp-wide: rows beyond the tile join in
        float v[16];
        tmem_ld16(tmem_o + lane_addr + d0, v);
        if (row_ok) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * e] * inv, v[2 * e + 1] * inv);
            w[e] = *reinterpret_cast<const uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(dst + d0) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + d0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      tc_fence_before();
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


// ---------------------------------------------------------------------------------------------
// Decode attention: the warp-level tensor-core kernel of attention_kernels.cuh with its key and
// value tiles brought by TMA instead of per-thread copies.  Per-thread loads (and cp.async)
// cannot keep enough bytes in flight per SM to fill HBM3e; a bulk tensor copy of a whole
// 16-key tile per instruction can.  One warp per (row, kv head x up to 8 query heads, split); each
// warp owns a ring of DSTAGES stages of 16 keys (K and V, two 64-dim chunks each, 128-byte
// swizzle) with one mbarrier per stage; lane 0 issues the copies, all lanes wait (bounded).
constexpr int DK = 16;            // keys per stage
constexpr int DSTAGES = 3;
constexpr int DSTAGE_BYTES = 2 * 2 * DK * 128;      // K and V, two chunks of 64 dims

struct DecodeParams {
  const __nv_bfloat16* q;
  const int* block_table;
  const int* pos;
  const int* slot;
  const int* row_list;
  __nv_bfloat16* out;
  float* scratch;
  int* error_flag;
  int* arrivals;     // one counter per (row, kv head, chunk of query heads), zero between launches; null: the
                     // pieces of an item are merged by a kernel of its own
  int n_rows, max_pages, page_size, nq, nkv, hd, window, split_keys, n_splits, g_chunks;
  int fresh_keys;    // at most this many of a row's newest keys (its own included) are written by the kernel before
  float scale;
  long long wait_cycles;     // limit of every wait on an mbarrier
  // Fused form (decoded tokens only): instead of q, the projection's output [qkv_slices][rows, (nq + 2 nkv) hd]
  // float32 (partial sums qkv_stride floats apart, plus qkv_bias), of which this kernel makes q (rotated), and the
  // row's new key (rotated) and value, which it writes into the cache and uses itself.
  const float* qkv;
  const float* qkv_bias;
  const float* cos_t;
  const float* sin_t;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int* page_error;
  long long qkv_stride;
  int qkv_slices, rot;
};

// Merge records [0, n_rec) of the ng query heads of one item, by a whole block of 128 threads:
// out = sum_s e^{m_s-M} o_s / sum_s e^{m_s-M} l_s, the records in order.  A thread takes pairs of output
// dims and fetches eight records at a time, all loads in flight together.  The records were written by other
// blocks: they are read past the first-level cache.
__device__ __forceinline__ void merge_records(const DecodeParams& p, int ti, int t, int h0, int ng, int n_rec) {
  const int hd = p.hd, rec = hd + 2, cols = hd >> 1;
  for (int pair = threadIdx.x; pair < ng * cols; pair += 128) {
    const int g = pair / cols, d = (pair % cols) * 2;
    const float* base = p.scratch + ((size_t)ti * p.nq + h0 + g) * p.n_splits * rec;
    float M = -INFINITY, L = 0.f;
    float2 acc = make_float2(0.f, 0.f);
    for (int s0 = 0; s0 < n_rec; s0 += 8) {
      float ms[8], ls[8];
      float2 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = s0 + u < n_rec;
        const float* r = base + (size_t)(in ? s0 + u : 0) * rec;
        ms[u] = in ? __ldcg(r + hd) : -INFINITY;
        ls[u] = in ? __ldcg(r + hd + 1) : 0.f;
        v[u] = in ? __ldcg(reinterpret_cast<const float2*>(r + d)) : make_float2(0.f, 0.f);
      }
      float Mn = M;
#pragma unroll
      for (int u = 0; u < 8; ++u) Mn = fmaxf(Mn, ms[u]);
      if (Mn > -INFINITY) {
        const float keep = M > -INFINITY ? expf(M - Mn) : 0.f;      // what was merged so far, on the new scale
        L *= keep;
        acc.x *= keep;
        acc.y *= keep;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (ms[u] > -INFINITY) {                                   // an empty record is left out
            const float w = expf(ms[u] - Mn);
            L += w * ls[u];
            acc.x += w * v[u].x;
            acc.y += w * v[u].y;
          }
        M = Mn;
      }
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    *reinterpret_cast<__nv_bfloat162*>(p.out + ((size_t)t * p.nq + h0 + g) * hd + d) =
        __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  }
}

// DKT: keys per stage of the ring, 16 or 32 (a stage of 32 keys is worked through as two halves of 16; it takes
// half as many copies and waits per key, and pages must be multiples of 32 keys)
// FUSED: the kernel also does the work of the rotary kernel for its rows (each one decoded token): the four warps
// of a block (four splits of one row and kv head) add up the projection's partial sums and the bias for the
// group's query heads, rotate them and keep q in shared memory; the block whose keys include the row's own position
// does the same for the new key and value, writes them into the cache page, and the warp that reaches that position
// puts them into its tile in shared memory (what the copy brought there is the page's old content).  So nothing
// in the cache that this kernel reads is written in this step, and every tile is asked for before the wait for the
// projection.
template <int HD, int DKT, bool FUSED>
__global__ void __launch_bounds__(128)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ DecodeParams p) {
  using flint_attn::ldsm4;
  using flint_attn::ldsm4t;
  using flint_attn::mma16816;
  constexpr int MG = 8;
  constexpr int SB = 2 * 2 * DKT * 128;        // bytes of a stage: K and V, two chunks of 64 dims
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[4 * DSTAGES];
  __shared__ __align__(16) float x_s[FUSED ? (MG + 2) * HD : 4];              // sums of 8 query heads, the key, the value
  __shared__ __align__(16) __nv_bfloat16 q_s[FUSED ? (MG + 2) * HD : 8];      // the same rotated and narrowed
  pdl_launch();
  // Nothing below reads what the kernels before this one write, until pdl_wait(): positions, slots and block
  // tables come from the host, and of the cache only a row's newest p.fresh_keys keys and values are written
  // in this step.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  const long long n_items = (long long)p.n_rows * p.nkv * p.g_chunks * p.n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % p.n_splits);
  long long rest = item / p.n_splits;
  const int gchunk = (int)(rest % p.g_chunks);
  rest /= p.g_chunks;
  const int kvh = (int)(rest % p.nkv);
  const int ti = (int)(rest / p.nkv);
  const int t = p.row_list ? p.row_list[ti] : ti;
  const int hd = p.hd, nq = p.nq;
  const int G = nq / p.nkv;
  const int g0 = gchunk * MG;
  const int ng = min(MG, G - g0);
  const int h0 = kvh * G + g0;
  const int pq = p.pos[t];
  const int lo_row = p.window > 0 ? max(0, pq + 1 - p.window) : 0;
  // the row's keys are divided evenly over the splits (in steps of 16), so that a row shorter than the
  // launch was sized for still keeps every split busy; split_keys is the upper bound
  const int even = ((pq + 1 - lo_row + p.n_splits - 1) / p.n_splits + DKT - 1) & ~(DKT - 1);
  const int sk = min(p.split_keys, max(even, DKT));
  const int lo = lo_row + split * sk;
  const int hi = min(pq + 1, lo + sk);
  const int* bt = p.block_table + (size_t)p.slot[t] * p.max_pages;
  const int gid = lane >> 2, tid4 = lane & 3;
  constexpr int KB = HD / 16, DB = HD / 8;
  const int kb_n = hd / 16, db_n = hd / 8, chunks = (hd + 63) / 64;

  const uint32_t ring = ((smem_u32(smem_raw) + 1023u) & ~1023u) + warp * (DSTAGES * SB);
  const uint32_t bar0 = smem_u32(&bars[warp * DSTAGES]);
  if (lane == 0) {
    for (int s = 0; s < DSTAGES; ++s) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  float o[DB][4];
#pragma unroll
  for (int db = 0; db < DB; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
  float m = -INFINITY, l = 0.f;

  // stages cover absolute key positions [first + step*16, +16): tiles never straddle a page
  const int first = lo & ~(DKT - 1);
  const int n_steps = hi > lo ? (hi - first + DKT - 1) / DKT : 0;
  auto issue = [&](int step, int stage) {      // lane 0 only
    const int j0 = first + step * DKT;
    const int lp = j0 / p.page_size;
    int page = lp < p.max_pages ? bt[lp] : -1;
    if (page < 0) page = 0;                    // never visible (masked): any finite page will do
    const int row = (page * p.nkv + kvh) * p.page_size + j0 % p.page_size;
    const uint32_t dst = ring + stage * SB, bar = bar0 + 8 * stage;
    mbar_expect_tx(bar, 2 * chunks * DKT * 128);
    for (int c = 0; c < chunks; ++c) {
      tma_load_2d(dst + c * DKT * 128, &map_k, c * 64, row, bar);
      tma_load_2d(dst + 2 * DKT * 128 + c * DKT * 128, &map_v, c * 64, row, bar);
    }
  };
  // the first tiles are asked for while the kernel before this one (which writes the newest keys and values, and
  // the queries) may still run; a tile that holds a key written in this step waits for it
  int issued = 0;
  if (lane == 0)
    for (; issued < DSTAGES - 1 && issued < n_steps &&
           (FUSED || first + (issued + 1) * DKT <= pq + 1 - p.fresh_keys); ++issued)
      issue(issued, issued);
  // the warp whose keys include the row's own position, and the step and row of its ring that hold it
  const bool owner_warp = FUSED && lo <= pq && hi == pq + 1;
  const int own_step = owner_warp ? (pq - first) / DKT : -1;
  // FUSED: what this warp prepares: two of the group's query heads, and, in the block that holds the split with
  // the row's own position, warp 0 the new key and warp 1 the new value.  A lane takes four neighbouring dims.
  // What does not come from the projection (bias, the rotation's cos and sin) is read before the wait for it.
  constexpr int JOBS = 3;
  const int d4 = lane * 4;
  int job_slot[JOBS], job_head[JOBS];
  bool job_on[JOBS];
  float4 job_bias[JOBS];
  float rc[4], rs[4];
  if (FUSED) {
    const int own_split = (pq - lo_row) / sk;
    const bool owner_block = (own_split >> 2) == (split >> 2);
    const int half = p.rot >> 1;
#pragma unroll
    for (int job = 0; job < JOBS; ++job) {
      if (job < 2) {
        const int g = warp * 2 + job;
        job_on[job] = g < ng && d4 < hd;
        job_slot[job] = g;
        job_head[job] = h0 + g;
      } else {
        job_on[job] = owner_block && warp < 2 && d4 < hd;
        job_slot[job] = MG + warp;
        job_head[job] = warp == 0 ? nq + kvh : nq + p.nkv + kvh;
      }
      job_bias[job] = (job_on[job] && p.qkv_bias)
                          ? *reinterpret_cast<const float4*>(p.qkv_bias + (size_t)job_head[job] * hd + d4)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int dd = d4 + e;
      rc[e] = 1.f;
      rs[e] = 0.f;
      if (dd < p.rot) {                              // dims i and i + rot/2 rotate together
        const int i = dd < half ? dd : dd - half;
        rc[e] = p.cos_t[(size_t)pq * half + i];
        rs[e] = p.sin_t[(size_t)pq * half + i];
      }
    }
  }
  pdl_wait();
  if (lane == 0)
    for (; issued < DSTAGES - 1 && issued < n_steps; ++issued) issue(issued, issued);
  if (FUSED) {
    const int half = p.rot >> 1;
    const size_t row_off = (size_t)t * (nq + 2 * p.nkv) * hd;
    // the partial sums of all of the warp's heads, five slices at a time in flight, added in order
    float4 acc[JOBS];
#pragma unroll
    for (int job = 0; job < JOBS; ++job) acc[job] = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int INFL = 5;
    for (int z0 = 0; z0 < p.qkv_slices; z0 += INFL) {
      float4 part[JOBS][INFL];
#pragma unroll
      for (int job = 0; job < JOBS; ++job)
#pragma unroll
        for (int u = 0; u < INFL; ++u)
          part[job][u] = (job_on[job] && z0 + u < p.qkv_slices)
                             ? *reinterpret_cast<const float4*>(p.qkv + (size_t)(z0 + u) * p.qkv_stride + row_off +
                                                                (size_t)job_head[job] * hd + d4)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int job = 0; job < JOBS; ++job)
#pragma unroll
        for (int u = 0; u < INFL; ++u) {
          acc[job].x += part[job][u].x; acc[job].y += part[job][u].y;
          acc[job].z += part[job][u].z; acc[job].w += part[job][u].w;
        }
    }
#pragma unroll
    for (int job = 0; job < JOBS; ++job)
      if (job_on[job]) {
        acc[job].x += job_bias[job].x; acc[job].y += job_bias[job].y;
        acc[job].z += job_bias[job].z; acc[job].w += job_bias[job].w;
        *reinterpret_cast<float4*>(&x_s[job_slot[job] * HD + d4]) = acc[job];
      }
    __syncwarp();                                    // a head's partner dims were summed by other lanes of this warp
#pragma unroll
    for (int job = 0; job < JOBS; ++job)
      if (job_on[job]) {
        const float* xr = &x_s[job_slot[job] * HD];
        const bool rotate = job < 2 || warp == 0;    // queries and the key; the value stays as it is
        const float own[4] = {acc[job].x, acc[job].y, acc[job].z, acc[job].w};
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int dd = d4 + e;
          y[e] = own[e];
          if (rotate && dd < p.rot)
            y[e] = dd < half ? own[e] * rc[e] - xr[dd + half] * rs[e] : own[e] * rc[e] + xr[dd - half] * rs[e];
        }
        const __nv_bfloat162 lo2 = __floats2bfloat162_rn(y[0], y[1]), hi2 = __floats2bfloat162_rn(y[2], y[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo2);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi2);
        *reinterpret_cast<uint2*>(&q_s[job_slot[job] * HD + d4]) = pk;
        if (job == 2 && gchunk == 0) {               // into the cache page, for the steps to come
          const int lp = pq / p.page_size;
          const int page = lp < p.max_pages ? bt[lp] : -1;
          if (page < 0) {
            if (lane == 0) atomicExch(p.page_error, 1);
          } else {
            __nv_bfloat16* dst = (warp == 0 ? p.k_cache : p.v_cache) +
                                 ((size_t)(page * p.nkv + kvh) * p.page_size + pq % p.page_size) * hd + d4;
            *reinterpret_cast<uint2*>(dst) = pk;
          }
        }
      }
    __syncthreads();
  }
  uint32_t qa[KB][2];
#pragma unroll
  for (int kb = 0; kb < KB; ++kb) {
    qa[kb][0] = qa[kb][1] = 0u;
    if (gid < ng && kb < kb_n) {
      const __nv_bfloat16* qp = FUSED ? &q_s[gid * HD + kb * 16 + tid4 * 2]
                                      : p.q + ((size_t)t * nq + h0 + gid) * hd + kb * 16 + tid4 * 2;
      qa[kb][0] = *reinterpret_cast<const uint32_t*>(qp);
      qa[kb][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }

  int failed = 0;
#pragma unroll 1
  for (int step = 0; step < n_steps; ++step) {
    const int stage = step % DSTAGES;
    __syncwarp();        // every lane is done reading the stage that is refilled next
    if (lane == 0 && step + DSTAGES - 1 < n_steps) issue(step + DSTAGES - 1, (step + DSTAGES - 1) % DSTAGES);
    {   // bounded wait for this stage's tile
      const uint32_t bar = bar0 + 8 * stage, parity = (step / DSTAGES) & 1;
      if (!mbar_try_wait(bar, parity)) {
        const long long t0 = clock64();
        while (!mbar_try_wait(bar, parity))
          if (clock64() - t0 > p.wait_cycles) { failed = 1; break; }
      }
    }
    if (__any_sync(0xffffffffu, failed)) break;
    if (FUSED && step == own_step) {
      // the row's own key and value: over what the copy brought from the page (its old content)
      const int r = pq - (first + step * DKT);
      for (int u = lane; u < 2 * (hd >> 3); u += 32) {            // 16-byte units of the key, then of the value
        const int is_v = u >= (hd >> 3), uu = is_v ? u - (hd >> 3) : u;
        const uint32_t dst = ring + stage * SB + is_v * 2 * DKT * 128 + (uu >> 3) * DKT * 128 + r * 128 +
                             (((uu & 7) ^ (r & 7)) << 4);
        const uint4 val = *reinterpret_cast<const uint4*>(&q_s[(MG + is_v) * HD + uu * 8]);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w)
                     : "memory");
      }
      __syncwarp();
    }
#pragma unroll
    for (int sub = 0; sub < DKT / 16; ++sub) {
    const uint32_t ks = ring + stage * SB + sub * 16 * 128, vs = ks + 2 * DKT * 128;
    const int j0 = first + step * DKT + sub * 16;
    float sacc[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
      for (int kb = 0; kb < KB; kb += 2) {
        if (kb < kb_n) {
          // matrices: this block's 8 keys x dims [kb*16, +8), [+8, +16), [(kb+1)*16, +8), [+8, +16)
          const int r = nb * 8 + (lane & 7);
          const int unit = kb * 2 + (lane >> 3);              // 16-byte unit along the head dimension
          uint32_t b0, b1, b2, b3;
          ldsm4(ks + (unit >> 3) * DKT * 128 + r * 128 + (((unit & 7) ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma16816(sacc[nb], qa[kb][0], 0u, qa[kb][1], 0u, b0, b1);
          if (kb + 1 < kb_n) mma16816(sacc[nb], qa[kb + 1][0], 0u, qa[kb + 1][1], 0u, b2, b3);
        }
      }
    }
    float sv[4];
    float mx = m;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = j0 + nb * 8 + tid4 * 2 + e;
        sv[nb * 2 + e] = (j >= lo && j < hi) ? sacc[nb][e] * p.scale : -INFINITY;
        mx = fmaxf(mx, sv[nb * 2 + e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float alpha = mx > -INFINITY ? expf(m - mx) : 1.f;
    m = mx;
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pv[i] = sv[i] > -INFINITY ? expf(sv[i] - mx) : 0.f;
    const __nv_bfloat162 p01 = __floats2bfloat162_rn(pv[0], pv[1]), p23 = __floats2bfloat162_rn(pv[2], pv[3]);
    l = l * alpha + ((__bfloat162float(p01.x) + __bfloat162float(p01.y)) + (__bfloat162float(p23.x) + __bfloat162float(p23.y)));
    const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&p01), pa2 = *reinterpret_cast<const uint32_t*>(&p23);
#pragma unroll
    for (int db = 0; db < DB; db += 2) {
      if (db < db_n) {
        o[db][0] *= alpha; o[db][1] *= alpha; o[db + 1][0] *= alpha; o[db + 1][1] *= alpha;
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;      // key row
        const int unit = db + (lane >> 4);                      // 16-byte unit = 8 dims
        uint32_t b0, b1, b2, b3;
        ldsm4t(vs + (unit >> 3) * DKT * 128 + r * 128 + (((unit & 7) ^ (r & 7)) << 4), b0, b1, b2, b3);
        mma16816(o[db], pa0, 0u, pa2, 0u, b0, b1);
        mma16816(o[db + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
    }
    }   // halves of a stage
  }
  if (failed && lane == 0) atomicExch(p.error_flag, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (p.n_splits == 1) {
    if (gid < ng && !failed) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)t * nq + h0 + gid) * hd + tid4 * 2;
#pragma unroll
      for (int db = 0; db < DB; ++db)
        if (db < db_n) *reinterpret_cast<__nv_bfloat162*>(dst + db * 8) = __floats2bfloat162_rn(o[db][0] * inv, o[db][1] * inv);
    }
    return;
  }
  if (failed) {            // an empty record: the merge leaves it out
    m = -INFINITY;
    l = 0.f;
  }
  const int rec = hd + 2;
  const int group = (int)(item / p.n_splits);
  if (!p.arrivals) {
    // one record per warp; a kernel of its own merges them
    if (gid < ng) {
      float* dst = p.scratch + (((size_t)ti * nq + h0 + gid) * p.n_splits + split) * rec;
#pragma unroll
      for (int db = 0; db < DB; ++db)
        if (db < db_n) { dst[db * 8 + tid4 * 2] = o[db][0]; dst[db * 8 + tid4 * 2 + 1] = o[db][1]; }
      if (tid4 == 0) { dst[hd] = m; dst[hd + 1] = l; }
    }
    return;
  }
  // The splits of an item come in fours, and the four warps of this block hold four consecutive splits of one
  // item: they merge through shared memory first, each warp taking two of the eight query heads, so that a
  // block leaves one record (or, with four splits in all, the result).
  __shared__ int s_failed[4];
  __shared__ int s_last;
  float* mine = reinterpret_cast<float*>(smem_raw + (ring - smem_u32(smem_raw)));    // this warp's ring, now free
  if (lane == 0) s_failed[warp] = failed;
  if (gid < ng && !failed) {
    float* dst = mine + gid * rec;
#pragma unroll
    for (int db = 0; db < DB; ++db)
      if (db < db_n) { dst[db * 8 + tid4 * 2] = o[db][0]; dst[db * 8 + tid4 * 2 + 1] = o[db][1]; }
    if (tid4 == 0) { dst[hd] = m; dst[hd + 1] = l; }
  }
  __syncthreads();
  const int n_rec = p.n_splits >> 2, rec_index = split >> 2;
  for (int g = warp * 2; g < min(warp * 2 + 2, ng); ++g) {
    const float* r4[4];
    float ms[4], M = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < 4; ++w2) {
      r4[w2] = reinterpret_cast<const float*>(smem_raw + (ring - smem_u32(smem_raw)) + (w2 - warp) * (DSTAGES * SB)) + g * rec;
      ms[w2] = s_failed[w2] ? -INFINITY : r4[w2][hd];
      M = fmaxf(M, ms[w2]);
    }
    float L = 0.f;
    float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
    for (int w2 = 0; w2 < 4; ++w2) {
      if (ms[w2] > -INFINITY) {
        const float wgt = expf(ms[w2] - M);
        L += wgt * r4[w2][hd + 1];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int d = lane * 2 + 64 * i;
          if (d < hd) {
            const float2 v = *reinterpret_cast<const float2*>(r4[w2] + d);
            acc[i].x += wgt * v.x;
            acc[i].y += wgt * v.y;
          }
        }
      }
    }
    if (n_rec == 1) {
      const float inv = L > 0.f ? 1.0f / L : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)t * nq + h0 + g) * hd;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int d = lane * 2 + 64 * i;
        if (d < hd) *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(acc[i].x * inv, acc[i].y * inv);
      }
    } else {
      float* dst = p.scratch + (((size_t)ti * nq + h0 + g) * p.n_splits + rec_index) * rec;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int d = lane * 2 + 64 * i;
        if (d < hd) *reinterpret_cast<float2*>(dst + d) = acc[i];
      }
      if (lane == 0) { dst[hd] = M; dst[hd + 1] = L; }
    }
  }
  if (n_rec == 1) return;
  // the block that arrives last of the item's blocks merges their records
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.arrivals + group, 1);
    s_last = prev == n_rec - 1;
    if (s_last) p.arrivals[group] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  merge_records(p, ti, t, h0, ng, n_rec);
}

// The same kernel with the work cut stream fashion: the 16-key steps of all (row, kv head, chunk of query
// heads) items, laid end to end, are divided into equal runs, one per warp of the grid, so that every warp
// reads the same number of keys whatever the rows' lengths are (a batch of requests of different lengths, a
// context shorter than the launch was sized for).  A warp's run may end one item and begin the next; each
// piece of an item goes to its own slot of the scratch records, in order, and the first piece marks the
// slots that the item does not use as empty (m = -inf, l = 0), so the merge needs no counts.
constexpr int MAX_STREAM_ROWS = 256;
constexpr int MIN_STREAM_STEPS = 3;      // a warp takes at least 48 keys

template <int HD>
__global__ void __launch_bounds__(128)
attention_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ DecodeParams p) {
  using flint_attn::ldsm4;
  using flint_attn::ldsm4t;
  using flint_attn::mma16816;
  constexpr int MG = 8;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[4 * DSTAGES];
  // units (steps of 16 keys x items of a row) before each row, and each row's steps: every warp works them
  // out for itself (a scan by shuffles), so that no warp waits for another before its first copy
  __shared__ int prefix_all[4][MAX_STREAM_ROWS + 1];
  __shared__ int steps_all[4][MAX_STREAM_ROWS];
  pdl_launch();
  // nothing below reads what the kernels before this one write, until pdl_wait() (see the kernel above)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* prefix = prefix_all[warp];
  int* steps_of = steps_all[warp];
  const int hd = p.hd, nq = p.nq;
  const int G = nq / p.nkv;
  const int ipr = p.nkv * p.g_chunks;               // items (kv head x chunk of query heads) per row
  int max_steps = 1, carried = 0;
  for (int base = 0; base < p.n_rows; base += 32) {
    const int ti = base + lane;
    int st = 0;
    if (ti < p.n_rows) {
      // steps of the row: its visible keys, from the 16-key boundary at or below the first one
      const int t = p.row_list ? p.row_list[ti] : ti;
      const int pq = p.pos[t];
      const int lo_row = p.window > 0 ? max(0, pq + 1 - p.window) : 0;
      st = (pq + 1 - (lo_row & ~(DK - 1)) + DK - 1) / DK;
      steps_of[ti] = st;
    }
    max_steps = max(max_steps, st);
    int incl = st * ipr;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (ti < p.n_rows) prefix[ti] = carried + incl - st * ipr;
    carried += __shfl_sync(0xffffffffu, incl, 31);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_steps = max(max_steps, __shfl_xor_sync(0xffffffffu, max_steps, o));
  if (lane == 0) prefix[p.n_rows] = carried;
  __syncwarp();
  const int total_units = carried;
  // equal runs of units, one per warp of the grid; long enough that an item has at most n_splits pieces
  const int n_warps = gridDim.x * 4;
  const int run_min = p.n_splits > 1 ? (max_steps - 1 + p.n_splits - 2) / (p.n_splits - 1) : max_steps;
  int run = max(max((total_units + n_warps - 1) / n_warps, run_min), MIN_STREAM_STEPS);
  if (p.n_splits == 1) run = ((run + max_steps - 1) / max_steps) * max_steps;
  const int w = blockIdx.x * 4 + warp;
  const long long u_begin = (long long)w * run;
  if (u_begin >= total_units) return;
  const int u_end = (int)min((long long)total_units, u_begin + run);
  const int gid = lane >> 2, tid4 = lane & 3;
  constexpr int KB = HD / 16, DB = HD / 8;
  const int kb_n = hd / 16, db_n = hd / 8, chunks = (hd + 63) / 64;

  const uint32_t ring = ((smem_u32(smem_raw) + 1023u) & ~1023u) + warp * (DSTAGES * DSTAGE_BYTES);
  const uint32_t bar0 = smem_u32(&bars[warp * DSTAGES]);
  if (lane == 0) {
    for (int s = 0; s < DSTAGES; ++s) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  int kc = 0;                       // stages issued so far by this warp: the rings run on across segments
  int failed = 0;
  bool waited = false;              // for the kernel before this one
  int ti = 0;
  for (int u = (int)u_begin; u < u_end && !failed;) {
    // the segment that starts at unit u: row, item of the row, first step
    while (prefix[ti + 1] <= u) ++ti;
    const int steps_row = steps_of[ti];
    const int rem = u - prefix[ti];
    const int j = rem / steps_row, s_begin = rem % steps_row;
    const int s_end = min(steps_row, s_begin + (u_end - u));
    const int kvh = j % p.nkv, gchunk = j / p.nkv;
    const int t = p.row_list ? p.row_list[ti] : ti;
    const int g0 = gchunk * MG;
    const int ng = min(MG, G - g0);
    const int h0 = kvh * G + g0;
    const int pq = p.pos[t];
    const int lo_row = p.window > 0 ? max(0, pq + 1 - p.window) : 0;
    const int first = lo_row & ~(DK - 1);
    const int lo = max(lo_row, first + s_begin * DK);
    const int hi = min(pq + 1, first + s_end * DK);
    const int* bt = p.block_table + (size_t)p.slot[t] * p.max_pages;
    // which piece of its item this segment is, and how many pieces the item has
    const int item_u0 = prefix[ti] + j * steps_row;
    const int first_w = item_u0 / run;
    const int piece = w - first_w;
    const int pieces = (item_u0 + steps_row - 1) / run - first_w + 1;
    float o[DB][4];
  #pragma unroll
    for (int db = 0; db < DB; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
    float m = -INFINITY, l = 0.f;

    // stages cover absolute key positions [first + step*16, +16): tiles never straddle a page
    const int n_steps = s_end - s_begin;
    auto issue = [&](int step, int stage) {      // lane 0 only
      const int j0 = first + (s_begin + step) * DK;
      const int lp = j0 / p.page_size;
      int page = lp < p.max_pages ? bt[lp] : -1;
      if (page < 0) page = 0;                    // never visible (masked): any finite page will do
      const int row = (page * p.nkv + kvh) * p.page_size + j0 % p.page_size;
      const uint32_t dst = ring + stage * DSTAGE_BYTES, bar = bar0 + 8 * stage;
      mbar_expect_tx(bar, 2 * chunks * DK * 128);
      for (int c = 0; c < chunks; ++c) {
        tma_load_2d(dst + c * DK * 128, &map_k, c * 64, row, bar);
        tma_load_2d(dst + 2 * DK * 128 + c * DK * 128, &map_v, c * 64, row, bar);
      }
    };
    __syncwarp();          // the previous segment's last reads of the ring are done
    // the warp's first tiles are asked for while the kernel before this one may still run, unless they hold a
    // key that it writes
    int issued = 0;
    if (lane == 0)
      for (; issued < DSTAGES - 1 && issued < n_steps &&
             (waited || first + (s_begin + issued + 1) * DK <= pq + 1 - p.fresh_keys); ++issued)
        issue(issued, (kc + issued) % DSTAGES);
    if (!waited) {
      pdl_wait();
      waited = true;
      if (lane == 0)
        for (; issued < DSTAGES - 1 && issued < n_steps; ++issued) issue(issued, (kc + issued) % DSTAGES);
    }
    uint32_t qa[KB][2];
  #pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      qa[kb][0] = qa[kb][1] = 0u;
      if (gid < ng && kb < kb_n) {
        const __nv_bfloat16* qp = p.q + ((size_t)t * nq + h0 + gid) * hd + kb * 16 + tid4 * 2;
        qa[kb][0] = *reinterpret_cast<const uint32_t*>(qp);
        qa[kb][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
    }

  #pragma unroll 1
    for (int step = 0; step < n_steps; ++step) {
      const int stage = (kc + step) % DSTAGES;
      __syncwarp();        // every lane is done reading the stage that is refilled next
      if (lane == 0 && step + DSTAGES - 1 < n_steps) issue(step + DSTAGES - 1, (kc + step + DSTAGES - 1) % DSTAGES);
      {   // bounded wait for this stage's tile
        const uint32_t bar = bar0 + 8 * stage, parity = ((kc + step) / DSTAGES) & 1;
        if (!mbar_try_wait(bar, parity)) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar, parity))
            if (clock64() - t0 > p.wait_cycles) { failed = 1; break; }
        }
      }
      failed = __any_sync(0xffffffffu, failed) ? 1 : 0;
      if (failed) break;
      const uint32_t ks = ring + stage * DSTAGE_BYTES, vs = ks + 2 * DK * 128;
      const int j0 = first + (s_begin + step) * DK;
      float sacc[2][4];
  #pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
  #pragma unroll
        for (int kb = 0; kb < KB; kb += 2) {
          if (kb < kb_n) {
            // matrices: this block's 8 keys x dims [kb*16, +8), [+8, +16), [(kb+1)*16, +8), [+8, +16)
            const int r = nb * 8 + (lane & 7);
            const int unit = kb * 2 + (lane >> 3);              // 16-byte unit along the head dimension
            uint32_t b0, b1, b2, b3;
            ldsm4(ks + (unit >> 3) * DK * 128 + r * 128 + (((unit & 7) ^ (r & 7)) << 4), b0, b1, b2, b3);
            mma16816(sacc[nb], qa[kb][0], 0u, qa[kb][1], 0u, b0, b1);
            if (kb + 1 < kb_n) mma16816(sacc[nb], qa[kb + 1][0], 0u, qa[kb + 1][1], 0u, b2, b3);
          }
        }
      }
      float sv[4];
      float mx = m;
  #pragma unroll
      for (int nb = 0; nb < 2; ++nb)
  #pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j0 + nb * 8 + tid4 * 2 + e;
          sv[nb * 2 + e] = (j >= lo && j < hi) ? sacc[nb][e] * p.scale : -INFINITY;
          mx = fmaxf(mx, sv[nb * 2 + e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float alpha = mx > -INFINITY ? expf(m - mx) : 1.f;
      m = mx;
      float pv[4];
  #pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = sv[i] > -INFINITY ? expf(sv[i] - mx) : 0.f;
      const __nv_bfloat162 p01 = __floats2bfloat162_rn(pv[0], pv[1]), p23 = __floats2bfloat162_rn(pv[2], pv[3]);
      l = l * alpha + ((__bfloat162float(p01.x) + __bfloat162float(p01.y)) + (__bfloat162float(p23.x) + __bfloat162float(p23.y)));
      const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&p01), pa2 = *reinterpret_cast<const uint32_t*>(&p23);
  #pragma unroll
      for (int db = 0; db < DB; db += 2) {
        if (db < db_n) {
          o[db][0] *= alpha; o[db][1] *= alpha; o[db + 1][0] *= alpha; o[db + 1][1] *= alpha;
          const int r = (lane & 7) + ((lane >> 3) & 1) * 8;      // key row
          const int unit = db + (lane >> 4);                      // 16-byte unit = 8 dims
          uint32_t b0, b1, b2, b3;
          ldsm4t(vs + (unit >> 3) * DK * 128 + r * 128 + (((unit & 7) ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma16816(o[db], pa0, 0u, pa2, 0u, b0, b1);
          mma16816(o[db + 1], pa0, 0u, pa2, 0u, b2, b3);
        }
      }
    }
    if (failed) break;
    kc += n_steps;
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (gid < ng) {
      float* dst = p.scratch + (((size_t)ti * nq + h0 + gid) * p.n_splits + piece) * (hd + 2);
#pragma unroll
      for (int db = 0; db < DB; ++db)
        if (db < db_n) { dst[db * 8 + tid4 * 2] = o[db][0]; dst[db * 8 + tid4 * 2 + 1] = o[db][1]; }
      if (tid4 == 0) { dst[hd] = m; dst[hd + 1] = l; }
      // the first piece marks the slots that the item has no piece for as empty
      if (piece == 0 && tid4 == 0)
        for (int z = pieces; z < p.n_splits; ++z) {
          float* e = p.scratch + (((size_t)ti * nq + h0 + gid) * p.n_splits + z) * (hd + 2);
          e[hd] = -INFINITY;
          e[hd + 1] = 0.f;
        }
    }
    u += n_steps;
  }
  if (failed && lane == 0) atomicExch(p.error_flag, 1);
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
  if (n_tiles > 65535 || nq > 0x7fffffff / 4) return fail("attention_tc: too many tiles or heads");
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
  p.wait_cycles = wait_limit();
  const int chunks = (hd + 63) / 64;
  const size_t smem = (size_t)chunks * BQ * 128 + (size_t)STAGES * 2 * chunks * BKV * 128;
  dim3 grid(nq, n_tiles);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    configured = true;
  }
  launch_pdl(attention_prefill_tc_kernel, grid, dim3(THREADS), smem, stream, mq, mk, mv, p);
  return check_launch("attention_prefill_tc");
}

// Decode rows (or any rows, one at a time) over the paged bfloat16 cache: the contract of
// flint_paged_attention with bfloat16 q/out, page sizes that are multiples of 16, head sizes up to 128.
// arrivals (may be null): n_arrivals counters, zero before the first launch and left zero by every launch;
// given enough of them and splits in fours, the splits of a row are merged inside this kernel.
// fresh_keys: how many of a row's newest keys (its own included) the kernel before this one in the stream may
// have written (1 for decoded tokens; the length of the longest portion otherwise): tiles below them are
// fetched before that kernel has finished.
static int launch_decode_tc(bool fused, DecodeParams& p, const void* k_cache, const void* v_cache, int n_pages,
                            int T, int nq, int nkv, int hd, int page_size, int split_keys, int n_splits, float* scratch,
                            const int* row_list, void* out, int* arrivals, int n_arrivals, cudaStream_t stream) {
  const char* who = fused ? "attention_decode_fused" : "attention_decode_tc";
  if (hd <= 0 || hd % 16 || hd > 128) return fail("%s: head size %d (multiples of 16 up to 128)", who, hd);
  if (nkv <= 0 || nq % nkv) return fail("%s: %d query heads do not divide into %d kv heads", who, nq, nkv);
  // Keys per stage: 32 for a row or two (one block of four warps per SM is then enough, and a stage of 32 keys
  // takes half as many copies and waits per key: -2.5 % of a decode step at batch 1), else 16, with which two
  // blocks share an SM (at batch 8 stages of 32 keys cost 8 % of the step)
  // (while its blocks fit one to an SM: a long context cut into more splits than that runs with stages of 16)
  const long long groups = (long long)T * nkv * ((nq / nkv + 7) / 8);
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const int dk = (page_size % 32 == 0 && groups <= 8 && groups * n_splits <= 4LL * sm_count) ? 32 : DK;
  if (page_size <= 0 || page_size % DK) return fail("%s: page size %d must be a multiple of %d", who, page_size, DK);
  if (n_splits < 1 || split_keys < 1) return fail("%s: bad split (%d keys, %d splits)", who, split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("%s: splits need scratch memory", who);
  if (!p.error_flag) return fail("%s: needs an error flag", who);
  CUtensorMap mk, mv;
  const long long kv_rows = (long long)n_pages * nkv * page_size;
  int rc = make_map_bf16(&mk, k_cache, kv_rows, hd, hd, dk);
  if (!rc) rc = make_map_bf16(&mv, v_cache, kv_rows, hd, hd, dk);
  if (rc) return fail("%s: cuTensorMapEncodeTiled failed (%d)", who, rc);
  p.row_list = row_list;
  p.out = (__nv_bfloat16*)out; p.scratch = scratch;
  p.n_rows = T; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd;
  p.split_keys = split_keys; p.n_splits = n_splits;
  p.g_chunks = (nq / nkv + 7) / 8;
  p.wait_cycles = wait_limit();
  // with splits in fours and a counter for every (row, kv head, chunk of query heads) the pieces are merged by
  // the block that finishes last; else by a kernel of its own
  p.arrivals = (arrivals && n_splits % 4 == 0 && (long long)T * nkv * p.g_chunks <= n_arrivals) ? arrivals : nullptr;
  if (fused && !p.arrivals)
    return fail("%s: needs splits in fours (got %d) and an arrival counter for each of the %lld items", who, n_splits,
                (long long)T * nkv * p.g_chunks);
  const long long items = (long long)T * nkv * p.g_chunks * n_splits;
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return fail("%s: too many work items", who);
  const size_t smem = (size_t)4 * DSTAGES * (2 * 2 * dk * 128) + 1024;
  static bool configured = false;
  if (!configured) {
    const int big = 4 * DSTAGES * (2 * 2 * 32 * 128) + 1024;
    cudaFuncSetAttribute(attention_decode_tc_kernel<64, 16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<128, 16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<64, 32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<128, 32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<64, 16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<128, 16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<64, 32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attention_decode_tc_kernel<128, 32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    configured = true;
  }
#define GO(H, D, F) launch_pdl(attention_decode_tc_kernel<H, D, F>, dim3((unsigned)blocks), dim3(128), smem, stream, mk, mv, p)
  if (fused) {
    if (dk == 32) { if (hd <= 64) GO(64, 32, true); else GO(128, 32, true); }
    else { if (hd <= 64) GO(64, 16, true); else GO(128, 16, true); }
  } else {
    if (dk == 32) { if (hd <= 64) GO(64, 32, false); else GO(128, 32, false); }
    else { if (hd <= 64) GO(64, 16, false); else GO(128, 16, false); }
  }
#undef GO
  rc = check_launch(who);
  if (rc || n_splits == 1 || p.arrivals) return rc;
  launch_pdl(flint_attn::attention_combine_kernel<__nv_bfloat16>, dim3((unsigned)((long long)T * nq)),
             dim3(hd >= 128 ? 128 : 64), 0, stream, (const float*)scratch, (__nv_bfloat16*)out, hd, n_splits, nq, row_list);
  return check_launch("attention_combine");
}

extern "C" int flint_attention_decode_tc(const void* q, const void* k_cache, const void* v_cache, int n_pages,
                                         const int* block_table, int max_pages, int page_size, const int* pos,
                                         const int* slot, void* out, int T, int nq, int nkv, int hd, int window,
                                         float scale, int split_keys, int n_splits, float* scratch,
                                         const int* row_list, int* error_flag, int* arrivals, int n_arrivals,
                                         int fresh_keys, cudaStream_t stream) {
  if (T <= 0) return 0;
  DecodeParams p = {};
  p.q = (const __nv_bfloat16*)q; p.block_table = block_table; p.pos = pos; p.slot = slot;
  p.error_flag = error_flag; p.max_pages = max_pages; p.window = window; p.scale = scale;
  p.fresh_keys = fresh_keys < 1 ? 1 : fresh_keys;
  return launch_decode_tc(false, p, k_cache, v_cache, n_pages, T, nq, nkv, hd, page_size, split_keys, n_splits, scratch,
                          row_list, out, arrivals, n_arrivals, stream);
}

// The decode kernel doing the rotary kernel's work as well, for rows that are one decoded token each (every row
// of the batch, no row list).  qkv [qkv_slices][T, (nq + 2 nkv) hd] float32: the q/k/v projection as partial
// sums qkv_stride floats apart, without its bias; bias [(nq + 2 nkv) hd] float32 or null; cos/sin
// [positions, rot/2] float32; q and k rotate over their first rot dims, dims i and i + rot/2 together.  The row's
// new key and value go into the cache (k_cache, v_cache: bfloat16 pages [page, nkv, page_size, hd]) and into the
// attention of this very launch.  n_splits must be a multiple of four and arrivals must hold a counter per
// (row, kv head, chunk of eight query heads).  page_error: set to 1 if a row's page is missing.
extern "C" int flint_attention_decode_fused(const float* qkv, int qkv_slices, long long qkv_stride, const float* bias,
                                            const float* cos_t, const float* sin_t, int rot, void* k_cache,
                                            void* v_cache, int n_pages, const int* block_table, int max_pages,
                                            int page_size, const int* pos, const int* slot, void* out, int T, int nq,
                                            int nkv, int hd, int window, float scale, int split_keys, int n_splits,
                                            float* scratch, int* error_flag, int* page_error, int* arrivals,
                                            int n_arrivals, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!qkv || qkv_slices < 1 || !cos_t || !sin_t || !page_error) return fail("attention_decode_fused: missing inputs");
  if (rot < 0 || rot > hd || (rot & 1)) return fail("attention_decode_fused: rotary size %d does not fit head size %d", rot, hd);
  if ((qkv_stride & 3) || ((uintptr_t)qkv & 15) || (bias && ((uintptr_t)bias & 15)))
    return fail("attention_decode_fused: the projection's rows must be 16-byte aligned");
  DecodeParams p = {};
  p.block_table = block_table; p.pos = pos; p.slot = slot;
  p.error_flag = error_flag; p.max_pages = max_pages; p.window = window; p.scale = scale;
  p.fresh_keys = 1;
  p.qkv = qkv; p.qkv_bias = bias; p.cos_t = cos_t; p.sin_t = sin_t; p.rot = rot;
  p.qkv_slices = qkv_slices; p.qkv_stride = qkv_stride;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache; p.page_error = page_error;
  return launch_decode_tc(true, p, k_cache, v_cache, n_pages, T, nq, nkv, hd, page_size, split_keys, n_splits, scratch,
                          nullptr, out, arrivals, n_arrivals, stream);
}

// The same contract with the work cut into equal runs of keys on the device (see the stream kernel): any mix of
// row lengths keeps every warp equally busy, and nothing about the launch depends on the lengths, so one
// captured launch serves every context length.  n_slices (2..64): the most pieces an item may be cut into;
// scratch: T * nq * n_slices * (hd + 2) floats.  Up to 256 rows.  fresh_keys: as for flint_attention_decode_tc.
extern "C" int flint_attention_decode_stream(const void* q, const void* k_cache, const void* v_cache, int n_pages,
                                             const int* block_table, int max_pages, int page_size, const int* pos,
                                             const int* slot, void* out, int T, int nq, int nkv, int hd, int window,
                                             float scale, int n_slices, float* scratch, const int* row_list,
                                             int* error_flag, int fresh_keys, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > MAX_STREAM_ROWS) return fail("attention_decode_stream: %d rows (up to %d)", T, MAX_STREAM_ROWS);
  if (hd <= 0 || hd % 16 || hd > 128) return fail("attention_decode_stream: head size %d (multiples of 16 up to 128)", hd);
  if (nkv <= 0 || nq % nkv) return fail("attention_decode_stream: %d query heads do not divide into %d kv heads", nq, nkv);
  if (page_size <= 0 || page_size % DK) return fail("attention_decode_stream: page size %d must be a multiple of %d", page_size, DK);
  if (n_slices < 2 || n_slices > 64) return fail("attention_decode_stream: %d slices (2..64)", n_slices);
  if (!scratch || !error_flag) return fail("attention_decode_stream: needs scratch memory and an error flag");
  CUtensorMap mk, mv;
  const long long kv_rows = (long long)n_pages * nkv * page_size;
  int rc = make_map_bf16(&mk, k_cache, kv_rows, hd, hd, DK);
  if (!rc) rc = make_map_bf16(&mv, v_cache, kv_rows, hd, hd, DK);
  if (rc) return fail("attention_decode_stream: cuTensorMapEncodeTiled failed (%d)", rc);
  DecodeParams p = {};
  p.q = (const __nv_bfloat16*)q; p.block_table = block_table; p.pos = pos; p.slot = slot; p.row_list = row_list;
  p.out = (__nv_bfloat16*)out; p.scratch = scratch; p.error_flag = error_flag;
  p.n_rows = T; p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd;
  p.window = window; p.split_keys = 0; p.n_splits = n_slices;
  p.g_chunks = (nq / nkv + 7) / 8;
  p.scale = scale;
  p.wait_cycles = wait_limit();
  p.arrivals = nullptr;
  p.fresh_keys = fresh_keys < 1 ? 1 : fresh_keys;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const size_t smem = 4 * DSTAGES * DSTAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_decode_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attention_decode_stream_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  const unsigned blocks = 2u * (unsigned)sm_count;           // two blocks of four warps stay resident per SM
  if (hd <= 64) launch_pdl(attention_decode_stream_kernel<64>, dim3(blocks), dim3(128), smem, stream, mk, mv, p);
  else launch_pdl(attention_decode_stream_kernel<128>, dim3(blocks), dim3(128), smem, stream, mk, mv, p);
  rc = check_launch("attention_decode_stream");
  if (rc) return rc;
  launch_pdl(flint_attn::attention_combine_kernel<__nv_bfloat16>, dim3((unsigned)((long long)T * nq)),
             dim3(hd >= 128 ? 128 : 64), 0, stream, (const float*)scratch, (__nv_bfloat16*)out, hd, n_slices, nq, row_list);
  return check_launch("attention_combine");
}

// The limit (clock cycles) that later launches of this module give their waits; 0 restores the default.
extern "C" void flint_attention_tc_set_wait_cycles(long long cycles) { wait_limit() = cycles > 0 ? cycles : WAIT_CYCLES; }

extern "C" const char* flint_attention_tc_last_error() { return g_error; }
