// bfloat16 matrix products on the 5th-generation tensor cores (tcgen05) of sm_100a:
//   out[r, n] = sum_k x[r, k] * W[n, k]      x [rows, K] bf16, W [N, K] bf16, fp32 accumulation.
//
// Layout of one CTA's tile.  The *weights* sit on the MMA's M side: a tile is 128 output
// features (rows of W) by BN token rows of x (BN = 16..256).  So the accumulator in tensor
// memory has one lane per output feature and one column per token, and small batches
// (decode) need no padding to 128 rows: a batch of 8 runs as a 128 x 16 tile that streams
// the weights once.  Both operands are K-major in shared memory, 64 bf16 (128 bytes) per
// row, 128-byte swizzle, loaded by TMA (cp.async.bulk.tensor.2d, no multicast); the
// K loop is a ring of `stages` buffers with full/empty mbarriers.
//
// Roles (192 threads): warp 0 lane 0 issues TMA loads; warp 1 allocates tensor memory and
// its lane 0 issues tcgen05.mma (4 of K=16 per 64-wide block) and tcgen05.commit; warps
// 2..5 wait for the accumulator, read it with tcgen05.ld (each warp its own 32 lanes) and
// run the epilogue: bias, SiLU/GELU gate times up, add to the output (residual stream),
// narrowing to bf16, or a float32 partial tile when the K range is split over several CTAs
// (then a second kernel sums the partials in a fixed order).
// A gated product (act(x Wg^T) * (x Wu^T)) takes its weights paired (blocks of 16 gate rows
// alternating with the 16 up rows of the same features), so a 128-row tile holds 64 features:
// one MMA per K step fills one accumulator whose lanes 0-15 of each warp's 32 hold gate values
// and lanes 16-31 the up values of the same 16 features, the epilogue pairs them with one
// shuffle, and the token tile can be as wide as for a plain product.
// Grouped products (experts) use the same kernel: rows are sorted by expert and a tile
// map names the expert and first row of each row tile; the experts' weights are one
// stacked [E*N, K] tensor, so a tile that hangs over the end of an expert reads rows
// of the next one and the epilogue masks them.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel sets an error
// flag, lets its copies land, frees its tensor memory and returns.
//
// Reference counterparts: crates/thuban_kernel/wgsl/gemm_coop_m16.wgsl (cooperative-matrix
// 16x16x16 tiles, f16), gemm.wgsl (ACC=1 residual add), gemv.wgsl (decode), bias.wgsl,
// swiglu.wgsl.
#include <cuda.h>
#include <math.h>
#include <stdarg.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tc_common.cuh"

using namespace flint;
using namespace flint_tc;

namespace {

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int GATED_FEATURES = BM / 2;   // gated: output features per tile (their gate rows and up rows)
static_assert(GATE_BLOCK == 16, "the gated epilogue pairs lanes l and l + 16 of a warp");
constexpr int BK = 64;           // bf16 per K block = one 128-byte swizzle row
constexpr int THREADS = 192;

struct Params {
  void* out;
  const float* bias;
  float* partial;              // [splits, rows, N] when splits > 1
  const int* tile_expert;
  const int* tile_row0;
  const int* n_tiles;
  const int* offsets;
  int* error_flag;
  int out_dtype, ldo, accumulate, act;
  int rows, N, K;
  int kb_per_split, splits, stages;
  int defer;                   // write raw partial tiles even for a single split; the consumer sums them
  int stream_k;                // cut the K blocks of all tiles, laid end to end, into equal runs, one per block
  int w_expert_rows;           // rows between two experts in the stacked weight tensor
  int plan_ready;              // grouped: the tile map was complete before this kernel could start (see flint_gemm_tc)
  long long wait_cycles;       // limit of every wait on an mbarrier
};
// Measured: with 232 bytes of parameters the compiler addressed them through a pointer and reloaded them after
// every store of the epilogue; the expert down product of a 2,048-token prefill ran 44 % slower.  Further
// parameters go into a second kernel argument.
static_assert(sizeof(Params) <= 128, "keep the parameter struct within 128 bytes");

// Instruction descriptor, kind::f16: fp32 accumulator, bf16 A and B, both K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t instr_desc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ float act_fn(float g, int act) {
  if (act == 0) return g / (1.0f + __expf(-g));
  return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// Persistent: a block walks over work items (feature tile, row tile, piece of K) with a stride of the
// grid.  The TMA ring runs on across items, and the accumulator is double-buffered in tensor memory, so
// the epilogue of one item overlaps the main loop of the next.
template <int BN, bool GATED>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * 16 + 4];   // full[stages], empty[stages], acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  // A product over experts that reads its tile map straight from the kernel that made it lets its own dependents
  // start only after it has waited for that kernel (below): whatever starts after it may then read the map at once.
  const bool grouped = p.tile_expert != nullptr;
  const bool map_pending = grouped && !p.plan_ready;
  if (!map_pending) pdl_launch();
  if (*(volatile int*)p.error_flag) return;   // an earlier block gave up: do not queue up behind it
  constexpr int FM = GATED ? GATED_FEATURES : BM;      // output features per tile
  const int tiles_m = (p.N + FM - 1) / FM;
  const int total_kb = (p.K + BK - 1) / BK;

  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = BN;                                      // columns of one accumulator set
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;  // two sets; a power of two
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stages = p.stages;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[16]);
  const uint32_t acc_full0 = smem_u32(&bars[32]), acc_empty0 = smem_u32(&bars[34]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 128);     // every epilogue thread arrives
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  volatile int* ab = &abort_flag;

  // The barriers and the tensor memory above need nothing from earlier kernels.  With experts, the tile map
  // comes from the routing plan of an earlier kernel: from here on the block has to wait for it, unless the
  // caller vouches that the map was complete before this kernel could start (an earlier product over the same
  // plan waited for it before it let anything after it start); then the weights of the first ring are on their
  // way while the kernel before this one still writes the rows.
  if (map_pending) {
    pdl_wait();
    pdl_launch();
  }
  const int tiles_n = grouped ? *p.n_tiles : (p.rows + BN - 1) / BN;
  const int n_items = tiles_m * tiles_n * p.splits;
  // Stream-K (few rows, partial sums deferred to the consumer): the K blocks of all tiles are laid end to end
  // and cut into runs of `run` blocks, one run per block of the grid, so that every block streams the same
  // number of weight bytes however many tiles there are (with experts, the number of tiles is only known
  // here).  A tile is then covered by up to p.splits pieces (run is kept long enough for that); piece i
  // of a tile goes to partial slice i, and the first piece also clears the slices the tile does not use.
  // A block without work (unit0 == unit1, or no item of its own) goes straight to the teardown.
  int run = 1, unit0 = 0, unit1 = 0;
  if (p.stream_k) {
    const long long units = (long long)tiles_m * tiles_n * total_kb;
    const int run_min = p.splits > 1 ? (total_kb - 1 + p.splits - 2) / (p.splits - 1) : total_kb;
    run = max(max((int)((units + gridDim.x - 1) / gridDim.x), run_min), 1);
    if (p.splits == 1) run = ((run + total_kb - 1) / total_kb) * total_kb;     // whole tiles only
    const long long u0 = (long long)blockIdx.x * run;
    if (u0 < units) {
      unit0 = (int)u0;
      unit1 = (int)min(units, u0 + run);
    }
  }

  // item -> (piece of K, feature tile, row tile): pieces of one tile and neighbouring feature tiles go
  // to neighbouring blocks, which then share the activation tile in L2
  // A tile that holds fewer than BN token rows (the end of an expert's rows, or of the batch) runs its MMAs
  // with N = its rows rounded up to 16.
  struct Item { int kb0, nkb, f0, w_row, row0, row_end, z, mma_n, pieces; bool valid; };
  // the j-th item of this block; not valid when it has no more
  auto item_at = [&](int j) -> Item {
    Item r;
    r.valid = false;
    int t;
    if (p.stream_k) {
      t = unit0 / total_kb + j;
      const int t_begin = t * total_kb;
      if (t_begin >= unit1) return r;
      r.kb0 = max(unit0, t_begin) - t_begin;
      r.nkb = min(unit1, t_begin + total_kb) - t_begin - r.kb0;
      const int first_block = t_begin / run;
      r.z = (int)blockIdx.x - first_block;
      r.pieces = (t_begin + total_kb - 1) / run - first_block + 1;
    } else {
      const int it = blockIdx.x + j * gridDim.x;
      if (it >= n_items) return r;
      r.z = it % p.splits;
      t = it / p.splits;
      r.kb0 = r.z * p.kb_per_split;
      r.nkb = min(total_kb, r.kb0 + p.kb_per_split) - r.kb0;
      r.pieces = p.splits;
    }
    const int tm = t % tiles_m, tn = t / tiles_m;
    int expert = 0;
    r.row0 = tn * BN;
    r.row_end = p.rows;
    if (grouped) {
      expert = p.tile_expert[tn];
      r.row0 = p.tile_row0[tn];
      r.row_end = p.offsets[expert + 1];
    }
    r.f0 = tm * FM;
    r.w_row = expert * p.w_expert_rows + tm * BM;
    const int valid = max(1, min(BN, r.row_end - r.row0));
    r.mma_n = (valid + 15) & ~15;
    r.valid = true;
    return r;
  };

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer
    int kc = 0;                      // K blocks issued so far, over all items
    bool first = true, ok = true;
    for (int j = 0; ok; ++j) {
      const Item w = item_at(j);
      if (!w.valid) break;
      int i = 0;
      if (first) {
        // The weights do not depend on the kernel before this one: the first ring of weight tiles is
        // requested at once, and only the activation tiles wait for that kernel to finish.
        const int head = w.nkb < stages ? w.nkb : stages;
        for (; i < head; ++i) {
          const uint32_t a = tiles + i * STAGE_BYTES, bar = full0 + 8 * i;
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(a, &map_w, (w.kb0 + i) * BK, w.w_row, bar);
        }
        pdl_wait();
        for (int j = 0; j < head; ++j)
          tma_load_2d(tiles + j * STAGE_BYTES + A_BYTES, &map_x, (w.kb0 + j) * BK, w.row0, full0 + 8 * j);
        kc = head;
        first = false;
      }
      for (; i < w.nkb; ++i, ++kc) {
        const int s = kc % stages;
        if (!mbar_wait(empty0 + 8 * s, ((kc / stages) & 1) ^ 1, ab, p.wait_cycles)) { ok = false; break; }
        const uint32_t a = tiles + s * STAGE_BYTES, bar = full0 + 8 * s;
        mbar_expect_tx(bar, STAGE_BYTES);
        const int kx = (w.kb0 + i) * BK;
        tma_load_2d(a, &map_w, kx, w.w_row, bar);
        tma_load_2d(a + A_BYTES, &map_x, kx, w.row0, bar);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    int kc = 0, j = 0;
    bool ok = true;
    for (; ok; ++j) {
      const Item w = item_at(j);
      if (!w.valid) break;
      const int buf = j & 1;
      ok = mbar_wait(acc_empty0 + 8 * buf, ((j >> 1) & 1) ^ 1, ab, p.wait_cycles);     // the epilogue has drained this set
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc_addr = tmem + buf * ACC_COLS;
      const uint32_t idesc = instr_desc(w.mma_n);
      for (int i = 0; i < w.nkb; ++i, ++kc) {
        const int s = kc % stages;
        ok = mbar_wait(full0 + 8 * s, (kc / stages) & 1, ab, p.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = tiles + s * STAGE_BYTES;
        const uint32_t b = a + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(acc_addr, smem_desc(a + k * 32), smem_desc(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);   // frees the stage when these MMAs have read it
      }
      if (ok) umma_commit(acc_full0 + 8 * buf);
    }
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // this warp's quarter of the 128 lanes
    const bool raw = p.splits > 1 || p.defer;     // partial tile: no bias, no accumulate
    bool waited = false;
    int j = 0;
    for (;; ++j) {
      const Item w = item_at(j);
      if (!w.valid) break;
      const int buf = j & 1;
      if (!mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1, ab, p.wait_cycles)) break;
      tc_fence_after();
      if (!waited) { pdl_wait(); waited = true; }   // before reading or writing what earlier kernels touch
      // output feature of this thread: its lane of the accumulator, or, gated, one of the warp's 16
      // features (lanes 0-15 hold its gate values, lanes 16-31 its up values)
      const int f = GATED ? w.f0 + q * GATE_BLOCK + (lane & 15) : w.f0 + q * 32 + lane;
      const bool f_ok = f < p.N;
      const float bias = (p.bias && f_ok && !raw) ? p.bias[f] : 0.f;
      const uint32_t lane_addr = tmem + buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
      constexpr int CH = BN < 32 ? 16 : 32;         // columns fetched from tensor memory at a time
#pragma unroll 1
      for (int c1 = 0; c1 < BN; c1 += CH) {
        if (w.row0 + c1 >= w.row_end) break;        // uniform in the warp
        float vv[CH];
        if (CH == 16) tmem_ld16(lane_addr + c1, vv); else tmem_ld32(lane_addr + c1, vv);
#pragma unroll
        for (int g = 0; g < CH; g += 8) {
          const int c0 = c1 + g;
          float* v = vv + g;
          if (GATED) {
            // the low half-warp takes token columns 0-3 and needs their up values, the high half takes
            // columns 4-7 and needs their gate values: one exchange of four values each
            const bool low = lane < 16;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float got = __shfl_xor_sync(0xffffffffu, low ? v[4 + c] : v[c], 16);
              const float gate = low ? v[c] : got, up = low ? got : v[4 + c];
              v[c] = act_fn(gate, p.act) * up;
            }
          }
#pragma unroll
          for (int c = 0; c < (GATED ? 4 : 8); ++c) {
            const int r = w.row0 + c0 + (GATED && lane >= 16 ? 4 + c : c);
            if (r >= w.row_end || !f_ok) continue;
            float y = v[c];
            if (raw) {
              p.partial[((size_t)w.z * p.rows + r) * p.N + f] = y;
              continue;
            }
            y += bias;
            const size_t o = (size_t)r * p.ldo + f;
            if (p.out_dtype == FLINT_F32) {
              float* out = (float*)p.out;
              out[o] = p.accumulate ? out[o] + y : y;
            } else {
              __nv_bfloat16* out = (__nv_bfloat16*)p.out;
              out[o] = __float2bfloat16_rn(p.accumulate ? __bfloat162float(out[o]) + y : y);
            }
          }
        }
      }
      // stream-K: the first piece of a tile clears the partial slices that the tile has no piece for
      if (raw && w.z == 0 && w.pieces < p.splits && f_ok)
        for (int r = w.row0; r < min(w.row_end, w.row0 + BN); ++r)
          for (int z = w.pieces; z < p.splits; ++z) p.partial[((size_t)z * p.rows + r) * p.N + f] = 0.f;
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
    }
  }
  // ---- teardown: everyone meets, tensor memory is freed by the warp that took it
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) {
      atomicExch(p.error_flag, 1);
      const long long t0 = clock64();     // let copies in flight land before the block ends
      while (clock64() - t0 < 200000) {}
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// out[r, f] = sum_z partial[z, r, f] (+ bias[f]) (+ out[r, f])
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int rows, int N,
                                     const float* __restrict__ bias, void* __restrict__ out, int out_dtype,
                                     int ldo, int accumulate) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * N) return;
  const int r = (int)(i / N), f = (int)(i % N);
  float y = 0.f;
  for (int z = 0; z < splits; ++z) y += partial[(size_t)z * rows * N + i];
  if (bias) y += bias[f];
  const size_t o = (size_t)r * ldo + f;
  if (out_dtype == FLINT_F32) {
    float* po = (float*)out;
    po[o] = accumulate ? po[o] + y : y;
  } else {
    __nv_bfloat16* po = (__nv_bfloat16*)out;
    po[o] = __float2bfloat16_rn(accumulate ? __bfloat162float(po[o]) + y : y);
  }
}

// ------------------------------------------------------------------ host: tensor maps
// 2-D bf16 tensor [rows, K] with a row stride of ld elements; box = 64 x box_rows, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* ptr, long long rows, int K, long long ld, int box_rows) {
  const int r = make_map_bf16(m, ptr, rows, K, ld, box_rows);
  if (r == -1) return fail("gemm_tc: cuTensorMapEncodeTiled is not available from the driver");
  if (r != 0) return fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d", r);
  return 0;
}

struct MapKey {
  const void* ptr; long long rows; int K; int box;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && box == o.box; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)k.K * 131 ^ (size_t)k.box;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_weight_maps;   // weights never move: encode once

int weight_map(CUtensorMap* m, const void* ptr, long long rows, int K, int box_rows = BM) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapKey key{ptr, rows, K, box_rows};
  auto it = g_weight_maps.find(key);
  if (it == g_weight_maps.end()) {
    CUtensorMap fresh;
    if (int rc = make_map(&fresh, ptr, rows, K, K, box_rows)) return rc;
    if (g_weight_maps.size() > 4096) g_weight_maps.clear();
    it = g_weight_maps.emplace(key, fresh).first;
  }
  *m = it->second;
  return 0;
}

template <int BN, bool GATED>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t stream) {
  constexpr int stage_bytes = BM * BK * 2 + BN * BK * 2;
  const size_t smem = (size_t)p.stages * stage_bytes + 1024;
  static bool configured = false;   // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return fail("gemm_tc: cannot raise shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  // persistent grid: at most as many blocks as stay resident (two per SM if shared memory and tensor
  // memory allow it), each walking over its share of the items
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  constexpr int acc_cols = 2 * BN;
  const int per_sm = (smem <= 74 * 1024 && acc_cols <= 128) ? 3 : (smem <= 110 * 1024 && acc_cols <= 256) ? 2 : 1;
  // stream-K: the work is cut into as many runs as blocks stay resident (at least one K block each)
  const long long items = p.stream_k ? (long long)grid.x * grid.y * ((p.K + BK - 1) / BK)
                                     : (long long)grid.x * grid.y * grid.z;
  const unsigned blocks = (unsigned)(items < (long long)sm_count * per_sm ? items : (long long)sm_count * per_sm);
  launch_pdl(gemm_tc_kernel<BN, GATED>, dim3(blocks), dim3(THREADS), smem, stream, mw, mx, p);
  return check_launch("gemm_tc");
}

}  // namespace

// Stages of the K ring for a token tile of bn rows: as many as fit about 100 KB (two blocks
// per SM), at least 3, at most 8 (wide tiles take up to 192 KB and run one block per SM).
static int g_stage_override = 0;
// For tuning: force the number of stages (0 = choose by tile size).
extern "C" void flint_gemm_tc_set_stages(int stages) { g_stage_override = stages; }

extern "C" int flint_gemm_tc_stages(int bn, int gated) {
  (void)gated;   // a gated tile has the same footprint: 64 gate and 64 up rows on the M side
  if (g_stage_override > 0 && bn < 128) return g_stage_override;   // tuning applies to the few-row tiles
  const int stage = BM * BK * 2 + bn * BK * 2;
  int s = (bn >= 128 ? 192 * 1024 : 100 * 1024) / stage;
  if (s < 3) s = 3;
  while (s * stage > 192 * 1024) --s;
  return s > 8 ? 8 : s;
}

// Floats of scratch needed for a K split.
extern "C" long long flint_gemm_tc_partial_floats(int rows, int N, int splits) {
  return splits > 1 ? (long long)splits * rows * N : 0;
}

// x [rows, K] bf16 with row stride ldx; w [E, N, K] bf16 (E = 1 when dense), or, gated, [E, paired_rows(N), K]
// with each expert's gate and up rows paired in blocks; out [rows, N].
// bn: token rows per tile (16, 32, 64, 128 or 256); with a tile map it must equal the plan's tile size.
// splits > 1 divides the K blocks over several CTAs and needs `partial` (not with a gated product).
// defer: leave the raw partial sums [splits, rows, N] in `partial` (no bias, nothing added to out);
// the caller's next kernel adds them up.
// stream_k (with defer): instead of splits equal pieces per tile, the K blocks of all tiles laid end to end are
// cut into equal runs, one per resident block; a tile gets at most `splits` pieces and every one of the
// `splits` slices of `partial` is written (pieces that do not exist as zeros).  The number of splits used is ceil(kb / ceil(kb / splits))
// with kb = ceil(K / 64).
// plan_ready (with a tile map): the map was written by a kernel that is certain to have finished when this one
// starts, because a product over the same map ran between the two (it lets its dependents start only after its
// own wait for the map's kernel); the first weight tiles are then fetched before the wait for the kernel before.
// error_flag: device int, set to 1 if a bounded wait ran out.
extern "C" int flint_gemm_tc(const void* x, int ldx, const void* w, int gated, const float* bias, void* out,
                             int out_dtype, int ldo, int accumulate, int act, const int* tile_expert,
                             const int* tile_row0, const int* n_tiles, const int* offsets, int max_tiles,
                             int n_experts, int rows, int N, int K, int bn, int splits, float* partial,
                             int defer, int stream_k, int plan_ready, int* error_flag, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7)) return fail("gemm_tc: K=%d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  if (ldx < K || (ldx & 7)) return fail("gemm_tc: row stride %d must be a multiple of 8 and at least K", ldx);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail("gemm_tc: operands must be 16-byte aligned");
  const bool w_up = gated != 0;
  const int w_expert_rows = gated ? paired_rows(N) : N;
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return fail("gemm_tc: bad token tile %d", bn);
  if (splits < 1) return fail("gemm_tc: bad split %d", splits);
  if ((splits > 1 || defer) && (w_up || !partial)) return fail("gemm_tc: partial sums need scratch and cannot be gated");
  if (!error_flag) return fail("gemm_tc: needs an error flag");
  if (stream_k && !defer) return fail("gemm_tc: stream-K leaves partial sums and needs defer");
  const int total_kb = (K + BK - 1) / BK;
  if (splits > total_kb) splits = total_kb;
  const int kbps = (total_kb + splits - 1) / splits;
  if (!stream_k) splits = (total_kb + kbps - 1) / kbps;            // no empty split
  const int tiles_n = tile_expert ? max_tiles : (rows + bn - 1) / bn;
  if (tiles_n <= 0) return 0;

  CUtensorMap mw, mx;
  if (int rc = weight_map(&mw, w, (long long)n_experts * w_expert_rows, K)) return rc;
  if (int rc = make_map(&mx, x, rows, K, ldx, bn)) return rc;

  Params p;
  p.out = out; p.bias = bias; p.partial = partial;
  p.tile_expert = tile_expert; p.tile_row0 = tile_row0; p.n_tiles = n_tiles; p.offsets = offsets;
  p.error_flag = error_flag;
  p.out_dtype = out_dtype; p.ldo = ldo; p.accumulate = accumulate; p.act = act;
  p.rows = rows; p.N = N; p.K = K;
  p.kb_per_split = kbps; p.splits = splits; p.defer = defer; p.stream_k = stream_k;
  p.w_expert_rows = w_expert_rows;
  p.plan_ready = (tile_expert && plan_ready) ? 1 : 0;
  p.wait_cycles = wait_limit();
  p.stages = flint_gemm_tc_stages(bn, w_up ? 1 : 0);
  // few rows: the product streams its weights and is bound by how many bytes an SM keeps in flight and by how
  // evenly the tiles spread; four stages of 18 KB let three blocks share an SM (444 resident blocks)
  if (bn < 64 && g_stage_override == 0 && p.stages > 4) p.stages = 4;
  if (p.stages > total_kb && total_kb >= 2) p.stages = total_kb;
  dim3 grid(w_up ? (N + GATED_FEATURES - 1) / GATED_FEATURES : (N + BM - 1) / BM, tiles_n, splits);
  int rc;
#define CASE(B)                                                                             \
  case B:                                                                                   \
    rc = w_up ? launch<B, true>(mw, mx, p, grid, stream) : launch<B, false>(mw, mx, p, grid, stream); \
    break;
  switch (bn) {
    CASE(16) CASE(32) CASE(64) CASE(128) CASE(256)
    default: rc = fail("gemm_tc: bad token tile %d", bn);
  }
#undef CASE
  if (rc || splits == 1 || defer) return rc;
  const size_t n = (size_t)rows * N;
  splitk_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(partial, splits, rows, N, bias, out,
                                                                        out_dtype, ldo, accumulate);
  return check_launch("gemm_tc split reduce");
}

// ------------------------------------------------------------------ the bounded wait by itself
// One thread waits, with the given limit, on an mbarrier at which nobody ever arrives: the wait runs out, the
// thread raises the error flag exactly as the product kernels do when a wait of theirs runs out, and the kernel
// returns.  Nothing faults and nothing hangs; tests use it to see the whole path from a wait that gave up to
// the host's error and back to a working engine.
__global__ void wait_probe_kernel(long long limit, int* error_flag) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, limit)) atomicExch(error_flag, 1);
  }
}

extern "C" int flint_gemm_tc_wait_probe(long long limit_cycles, int* error_flag, cudaStream_t stream) {
  if (limit_cycles < 1 || limit_cycles > WAIT_CYCLES) return fail("wait probe: the limit must be 1..%lld cycles", WAIT_CYCLES);
  if (!error_flag) return fail("wait probe: needs an error flag");
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_cycles, error_flag);
  return check_launch("wait probe");
}

// The limit (clock cycles) that later launches of this module give their waits; 0 restores the default.
extern "C" void flint_gemm_tc_set_wait_cycles(long long cycles) { wait_limit() = cycles > 0 ? cycles : WAIT_CYCLES; }

extern "C" const char* flint_gemm_tc_last_error() { return g_error; }
