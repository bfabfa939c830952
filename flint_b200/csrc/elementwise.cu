// Row-wise kernels: embedding lookup, LayerNorm / RMSNorm, rotary position encoding
// fused with the write of keys and values into the paged cache, row gather, and the
// weighted sum of the two selected experts' outputs into the residual stream.
//
// Reference counterparts (WGSL, crates/thuban_kernel/wgsl/): embed.wgsl, norm.wgsl
// (mode 3 = LayerNorm with bias), rope.wgsl + kv_store.wgsl, add.wgsl.  All arithmetic
// is float32; only loads widen and stores narrow.
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

// --------------------------------------------------------------------------- embed
// fed_rows (may be null): for each row -1, or the place in `fed_from` (the sampler's last output, still on the
// device) that holds the row's token: a decoded token can be fed to the next step before the host has read it.
template <typename TT>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ fed_rows,
                             const int* __restrict__ fed_from, const TT* __restrict__ table,
                             float* __restrict__ out, int T, int H, int V, float scale) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int fed = fed_rows ? fed_rows[r] : -1;
  int id = fed >= 0 ? fed_from[fed] : ids[r];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);  // ids are validated on the host; never read outside
  const TT* src = table + (size_t)id * H;
  float* dst = out + (size_t)r * H;
  for (int d = threadIdx.x; d < H; d += blockDim.x) dst[d] = to_f32(src[d]) * scale;
}

extern "C" int flint_embed(const int* ids, const int* fed_rows, const int* fed_from, const void* table, int table_dtype,
                           float* out, int T, int H, int V, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) return fail("embed: bad sizes H=%d V=%d", H, V);
  if ((fed_rows == nullptr) != (fed_from == nullptr)) return fail("embed: fed rows and their source come together");
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  FLINT_DISPATCH_DTYPE(table_dtype, TT,
      launch_pdl(embed_kernel<TT>, dim3(T), dim3(threads), 0, stream, ids, fed_rows, fed_from, (const TT*)table, out, T,
                 H, V, scale));
  return check_launch("embed");
}

// --------------------------------------------------------------------------- norm
// mode 0: LayerNorm (x-mean)*rsqrt(var+eps)*gamma (+beta), var = mean((x-mean)^2)
// mode 1: RMSNorm   x*rsqrt(mean(x^2)+eps)*gamma
// One block per output row; statistics in float32 with three passes over the row (the
// row stays in L1 between passes).  row_index, if given, selects the input row.
__global__ void norm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            float eps, int mode, float* __restrict__ out_f32,
                            __nv_bfloat16* __restrict__ out_bf16, int H) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src_row = row_index ? row_index[r] : r;
  const float* xr = x + (size_t)src_row * H;
  float mean = 0.f;
  if (mode == 0) {
    float s = 0.f;
    for (int d = threadIdx.x; d < H; d += blockDim.x) s += xr[d];
    mean = block_sum(s, red) / (float)H;
  }
  float ss = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float c = xr[d] - mean;
    ss += c * c;
  }
  const float var = block_sum(ss, red) / (float)H;
  const float inv = 1.0f / sqrtf(var + eps);
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    float y = (xr[d] - mean) * inv * gamma[d];
    if (beta) y += beta[d];
    if (out_f32) out_f32[(size_t)r * H + d] = y;
    if (out_bf16) out_bf16[(size_t)r * H + d] = __float2bfloat16_rn(y);
  }
}

extern "C" int flint_norm(const float* x, const int* row_index, const float* gamma,
                          const float* beta, float eps, int mode, float* out_f32, void* out_bf16,
                          int rows, int H, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0) return fail("norm: bad width %d", H);
  if (mode != 0 && mode != 1) return fail("norm: unknown mode %d", mode);
  if (!out_f32 && !out_bf16) return fail("norm: no output given");
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  norm_kernel<<<rows, threads, 0, stream>>>(x, row_index, gamma, beta, eps, mode, out_f32,
                                            (__nv_bfloat16*)out_bf16, H);
  return check_launch("norm");
}

// four neighbouring values written with one store
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const uint32_t*>(&lo);
  w.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = w;
}

// --------------------------------------------------------------------------- rope + kv write
// qkv [n_partials][T, (nq+2*nkv)*hd] float32: q heads, then k heads, then v heads; the partials
// (pieces of a split K range, partial_stride floats apart) and the bias are added on the way in.
// q and k are rotated over the first `rot` dims of each head by the row of the cos/sin tables that belongs to
// the token's position: dims i and i + rot/2 together (NeoX half-split), or, interleaved, dims 2i and 2i + 1; q goes to q_out, k and v go to
// the token's place in the paged cache: page = block_table[slot, pos / P], row pos % P.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
rope_kv_kernel(const float* __restrict__ qkv, const int* __restrict__ pos,
                               const int* __restrict__ slot, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, int rot, int interleaved, TQ* __restrict__ q_out,
                               TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                               const int* __restrict__ block_table, int max_pages, int page_size,
                               int nq, int nkv, int hd, int write_kv, int* __restrict__ status,
                               int n_partials, long long partial_stride, const float* __restrict__ bias) {
  pdl_launch();
  // One block per token.  A work item is a pair of dims (d, d + rot/2) of one head (or two
  // neighbouring dims beyond the rotary part, or of a value head), so that every input element
  // is read exactly once; consecutive threads take consecutive pairs.
  // Positions, slots, block tables, the cos/sin tables and the bias are not written by any kernel: they are read
  // before the wait for the kernel before this one, whose output (qkv) is read only after it.
  const int t = blockIdx.x;
  const int p = pos[t];
  const int half = rot >> 1;
  const int pairs = hd >> 1;                 // per head
  const int heads = nq + (write_kv ? 2 * nkv : 0);
  const size_t row_off = (size_t)t * (nq + 2 * nkv) * hd;
  long long cache_tok = -1;                  // row of this token in [page, kv_head, P] units, head 0
  bool missing = false;
  if (write_kv) {
    const int page = block_table[(size_t)slot[t] * max_pages + p / page_size];
    if (page < 0) missing = true;            // the host must have allocated the page; record and skip
    else cache_tok = (long long)page * nkv * page_size + (p % page_size);
  }
  // with few tokens several blocks share a token (gridDim.y), each a contiguous range of items
  const int n_items = heads * pairs;
  const int per_block = (n_items + gridDim.y - 1) / gridDim.y;
  const int item_end = min(n_items, (int)(blockIdx.y + 1) * per_block);
  // fast path (head size and rotary size multiples of 8, 16-byte aligned pointers and slices): a thread
  // takes 4 neighbouring pairs with 16-byte loads
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(cos_t) |
                           reinterpret_cast<uintptr_t>(sin_t) | reinterpret_cast<uintptr_t>(bias) |
                           reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
                           reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  // (several blocks to a token only while each still has a block's worth of them: with 24 tokens and 13 blocks
  // each, the item-by-item path below is the faster)
  const int quads = pairs >> 2;
  const int q_per_block = (heads * quads + gridDim.y - 1) / gridDim.y;
  if ((half & 3) == 0 && (hd & 7) == 0 && aligned16 && !interleaved && (partial_stride & 3) == 0 &&
      (gridDim.y == 1 || q_per_block >= 128)) {
    pdl_wait();
    if (missing && threadIdx.x == 0 && blockIdx.y == 0) atomicExch(status, 1);
    const int q_end = min(heads * quads, (int)(blockIdx.y + 1) * q_per_block);
    for (int item = blockIdx.y * q_per_block + threadIdx.x; item < q_end; item += blockDim.x) {
      const int head = item / quads, i = (item % quads) * 4;      // first pair of the four
      const bool is_q = head < nq, is_v = head >= nq + nkv;
      int d0, d1;
      bool rotate = false;
      if (!is_v && i < half) { d0 = i; d1 = i + half; rotate = true; }
      else if (is_v) { d0 = 2 * i; d1 = 2 * i + 4; }               // eight neighbouring dims
      else { d0 = rot + 2 * (i - half); d1 = d0 + 4; }
      const size_t base = row_off + (size_t)head * hd;
      float4 x0 = *reinterpret_cast<const float4*>(qkv + base + d0);
      float4 x1 = *reinterpret_cast<const float4*>(qkv + base + d1);
      // further partial sums of the projection, four slices in flight at a time, added in order
      for (int z0 = 1; z0 < n_partials; z0 += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bool in = z0 + u < n_partials;
          const float* sl = qkv + (size_t)(in ? z0 + u : 0) * partial_stride + base;
          a[u] = in ? *reinterpret_cast<const float4*>(sl + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
          b[u] = in ? *reinterpret_cast<const float4*>(sl + d1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          x0.x += a[u].x; x0.y += a[u].y; x0.z += a[u].z; x0.w += a[u].w;
          x1.x += b[u].x; x1.y += b[u].y; x1.z += b[u].z; x1.w += b[u].w;
        }
      }
      if (bias) {
        const float4 b0 = *reinterpret_cast<const float4*>(bias + head * hd + d0);
        const float4 b1 = *reinterpret_cast<const float4*>(bias + head * hd + d1);
        x0.x += b0.x; x0.y += b0.y; x0.z += b0.z; x0.w += b0.w;
        x1.x += b1.x; x1.y += b1.y; x1.z += b1.z; x1.w += b1.w;
      }
      if (rotate) {
        const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)p * half + i);
        const float4 sn = *reinterpret_cast<const float4*>(sin_t + (size_t)p * half + i);
        const float4 y0 = make_float4(x0.x * c.x - x1.x * sn.x, x0.y * c.y - x1.y * sn.y, x0.z * c.z - x1.z * sn.z,
                                      x0.w * c.w - x1.w * sn.w);
        const float4 y1 = make_float4(x1.x * c.x + x0.x * sn.x, x1.y * c.y + x0.y * sn.y, x1.z * c.z + x0.z * sn.z,
                                      x1.w * c.w + x0.w * sn.w);
        x0 = y0;
        x1 = y1;
      }
      if (is_q) {
        TQ* dst = q_out + ((size_t)t * nq + head) * hd;
        store4(dst + d0, x0);
        store4(dst + d1, x1);
      } else if (cache_tok >= 0) {
        const int kvh = is_v ? head - nq - nkv : head - nq;
        TC* dst = (is_v ? v_cache : k_cache) + (cache_tok + (long long)kvh * page_size) * hd;
        store4(dst + d0, x0);
        store4(dst + d1, x1);
      }
    }
    return;
  }
  // what an item needs that no kernel writes: its dims, its cos and sin, its bias
  struct Item { int head, d0, d1; bool rotate; float c, s, b0, b1; };
  auto prepare = [&](int item) {
    Item it;
    it.head = item / pairs;
    const int i = item % pairs;
    const bool is_v = it.head >= nq + nkv;
    // dims of this item: inside the rotary part (d, d + half); beyond it (rot + 2j, rot + 2j + 1)
    it.rotate = false;
    if (!is_v && i < half) {
      it.d0 = interleaved ? 2 * i : i;
      it.d1 = interleaved ? 2 * i + 1 : i + half;
      it.rotate = true;
    }
    else if (is_v) { it.d0 = 2 * i; it.d1 = 2 * i + 1; }
    else { it.d0 = rot + 2 * (i - half); it.d1 = it.d0 + 1; }
    it.c = it.rotate ? cos_t[(size_t)p * half + i] : 1.f;
    it.s = it.rotate ? sin_t[(size_t)p * half + i] : 0.f;
    it.b0 = bias ? bias[it.head * hd + it.d0] : 0.f;
    it.b1 = bias ? bias[it.head * hd + it.d1] : 0.f;
    return it;
  };
  int item = blockIdx.y * per_block + threadIdx.x;
  Item it;
  if (item < item_end) it = prepare(item);
  pdl_wait();
  if (missing && threadIdx.x == 0) atomicExch(status, 1);
  while (item < item_end) {
    // the projection may arrive as partial sums over pieces of its K range, and without its bias: they are
    // added here in a fixed order (up to sixteen loads of each of the two values in flight)
    const float* s0 = qkv + row_off + (size_t)it.head * hd + it.d0;
    const float* s1 = qkv + row_off + (size_t)it.head * hd + it.d1;
    float x0 = 0.f, x1 = 0.f;
    for (int z0 = 0; z0 < n_partials; z0 += 16) {
      float t0[16], t1[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const bool in = z0 + u < n_partials;
        t0[u] = in ? s0[(size_t)(z0 + u) * partial_stride] : 0.f;
        t1[u] = in ? s1[(size_t)(z0 + u) * partial_stride] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) { x0 += t0[u]; x1 += t1[u]; }
    }
    x0 += it.b0;
    x1 += it.b1;
    if (it.rotate) {
      const float y0 = x0 * it.c - x1 * it.s, y1 = x1 * it.c + x0 * it.s;
      x0 = y0;
      x1 = y1;
    }
    const int head = it.head;
    const bool is_q = head < nq, is_v = head >= nq + nkv;
    if (is_q) {
      TQ* dst = q_out + ((size_t)t * nq + head) * hd;
      dst[it.d0] = from_f32<TQ>(x0);
      dst[it.d1] = from_f32<TQ>(x1);
    } else if (cache_tok >= 0) {
      const int kvh = is_v ? head - nq - nkv : head - nq;
      TC* dst = (is_v ? v_cache : k_cache) + (cache_tok + (long long)kvh * page_size) * hd;
      dst[it.d0] = from_f32<TC>(x0);
      dst[it.d1] = from_f32<TC>(x1);
    }
    item += blockDim.x;
    if (item < item_end) it = prepare(item);
  }
}

extern "C" int flint_rope_kv_write(const float* qkv, const int* pos, const int* slot,
                                   const float* cos_t, const float* sin_t, int rot, int interleaved, void* q_out,
                                   int q_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                   const int* block_table, int max_pages, int page_size, int T,
                                   int nq, int nkv, int hd, int write_kv, int* status,
                                   int n_partials, long long partial_stride, const float* bias,
                                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_partials < 1) return fail("rope: needs at least one partial");
  if (rot < 0 || rot > hd || (rot & 1)) return fail("rope: rotary size %d does not fit head size %d", rot, hd);
  if (page_size <= 0) return fail("rope: bad page size %d", page_size);
  const int items = (nq + 2 * nkv) * (hd / 2);
  int per_token = T >= 296 ? 1 : (296 + T - 1) / T;            // enough blocks to fill the device
  if (per_token > (items + 63) / 64) per_token = (items + 63) / 64;
  if (per_token < 1) per_token = 1;
  dim3 grid(T, per_token);
  const int share = (items + per_token - 1) / per_token;
  const int threads = share >= 256 ? 256 : ((share + 31) / 32) * 32;
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC,
      (launch_pdl(rope_kv_kernel<TQ, TC>, grid, dim3(threads), 0, stream,
          qkv, pos, slot, cos_t, sin_t, rot, interleaved, (TQ*)q_out, (TC*)k_cache, (TC*)v_cache, block_table,
          max_pages, page_size, nq, nkv, hd, write_kv, status, n_partials, partial_stride, bias))));
  return check_launch("rope_kv_write");
}

// --------------------------------------------------------------------------- row gather
// out[r, :] = x[index[r], :] for rows of row_bytes bytes (a multiple of 4); a negative
// index gives a row of zeros.
template <typename V>
__global__ void gather_rows_kernel(const V* __restrict__ x, const int* __restrict__ index,
                                   V* __restrict__ out, int words) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = index[r];
  V zero;
  memset(&zero, 0, sizeof(V));
  for (int d = threadIdx.x; d < words; d += blockDim.x)
    out[(size_t)r * words + d] = src < 0 ? zero : x[(size_t)src * words + d];
}

extern "C" int flint_gather_rows(const void* x, const int* index, void* out, int rows,
                                 int row_bytes, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (row_bytes <= 0 || (row_bytes & 3)) return fail("gather_rows: row size %d bytes is not a multiple of 4", row_bytes);
  // rows of whole 16-byte units that start on 16 bytes move in such units
  if ((row_bytes & 15) == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const int words = row_bytes / 16;
    launch_pdl(gather_rows_kernel<uint4>, dim3(rows), dim3(words >= 256 ? 256 : 128), 0, stream, (const uint4*)x, index,
               (uint4*)out, words);
  } else {
    launch_pdl(gather_rows_kernel<uint32_t>, dim3(rows), dim3(256), 0, stream, (const uint32_t*)x, index, (uint32_t*)out,
               row_bytes / 4);
  }
  return check_launch("gather_rows");
}

// --------------------------------------------------------------------------- expert combine
// h[t,:] += g[t,0]*y[row_of[t,0],:] + g[t,1]*y[row_of[t,1],:]   (always in this order)
__global__ void moe_combine_kernel(float* __restrict__ h, const float* __restrict__ y,
                                   const int* __restrict__ row_of, const float* __restrict__ gates,
                                   int H) {
  const int t = blockIdx.x;
  const int r0 = row_of[2 * t], r1 = row_of[2 * t + 1];
  const float g0 = gates[2 * t], g1 = gates[2 * t + 1];
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    float acc = g0 * y[(size_t)r0 * H + d];
    acc += g1 * y[(size_t)r1 * H + d];
    h[(size_t)t * H + d] += acc;
  }
}

extern "C" int flint_moe_combine(float* h, const float* y, const int* row_of, const float* gates,
                                 int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  moe_combine_kernel<<<T, 256, 0, stream>>>(h, y, row_of, gates, H);
  return check_launch("moe_combine");
}

// x[r, c] += sum_z partials[z][r, c] (+ bias[c]): the fallback for widths the fused row kernel refuses.
__global__ void add_partials_kernel(float* __restrict__ x, const float* __restrict__ partials, int n_partials,
                                    long long stride, const float* __restrict__ bias, long long n, int H) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i];
  for (int z = 0; z < n_partials; ++z) v += partials[(size_t)z * stride + i];
  if (bias) v += bias[i % H];
  x[i] = v;
}

extern "C" int flint_add_partials(float* x, const float* partials, int n_partials, long long stride,
                                  const float* bias, int rows, int H, cudaStream_t stream) {
  const long long n = (long long)rows * H;
  if (n <= 0) return 0;
  add_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, partials, n_partials, stride, bias, n, H);
  return check_launch("add_partials");
}

// out[r, i] = act(sum_z gate[z][r, i]) * sum_z up[z][r, i]: the epilogue of a gated product whose K range was
// split (p: [S, rows, paired_rows(I)] float32 partial sums, gate and up columns paired in blocks like the weight
// rows that made them).
template <typename TO>
__global__ void gated_act_kernel(const float* __restrict__ p, int S, long long stride, TO* __restrict__ out,
                                 int rows, int I, int act) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * I) return;
  const int r = (int)(i / I), c = (int)(i % I);
  float g = 0.f, u = 0.f;
  for (int z = 0; z < S; ++z) {
    const float* row = p + (size_t)z * stride + (size_t)r * paired_rows(I) + paired_gate_row(c);
    g += row[0];
    u += row[GATE_BLOCK];
  }
  const float a = act == 0 ? g / (1.0f + expf(-g))
                           : 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  out[i] = from_f32<TO>(a * u);
}

extern "C" int flint_gated_act(const float* partials, int S, long long stride, void* out, int out_dtype, int rows,
                               int I, int act, cudaStream_t stream) {
  const long long n = (long long)rows * I;
  if (n <= 0) return 0;
  if (S < 1) return fail("gated_act: needs at least one partial");
  FLINT_DISPATCH_DTYPE(out_dtype, TO,
      launch_pdl(gated_act_kernel<TO>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, partials, S, stride,
                 (TO*)out, rows, I, act));
  return check_launch("gated_act");
}

extern "C" const char* flint_elementwise_last_error() { return g_error; }
