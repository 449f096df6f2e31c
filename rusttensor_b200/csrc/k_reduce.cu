// Axis reductions (sum / mean / max / min / prod / logsumexp / argmax / argmin),
// log_softmax, and their gradients, over a tensor viewed as [outer, len, inner].
//
// inner == 1  (reduce contiguous rows): a warp per short row (shuffle reduction), a
//              256-thread block per long row (shared-memory reduction, 128-bit loads),
//              or, when there are few long rows, a split into chunks whose partial
//              results are reduced by a second pass.
// inner  > 1  (reduce a strided axis): threads run along `inner` (coalesced), rows of
//              the reduced axis are spread over threadIdx.y and, when the output is
//              small, over blockIdx.y with a second pass over the partials.
// Every multi-block reduction adds its partial results in a fixed order (a second pass,
// or the last block of a tile in split order; the only atomic is that block's ticket),
// so results are run-to-run deterministic.
#include <cfloat>
#include <cmath>
#include <mutex>

#include "rt_internal.cuh"

namespace {

constexpr int kThreads = 256;

template <int KIND>
struct Red;
template <>
struct Red<RT_RED_SUM> {
  static __device__ __forceinline__ float init() { return 0.f; }
  static __device__ __forceinline__ float op(float a, float b) { return a + b; }
};
template <>
struct Red<RT_RED_MAX> {
  static __device__ __forceinline__ float init() { return -INFINITY; }
  static __device__ __forceinline__ float op(float a, float b) { return fmaxf(a, b); }
};
template <>
struct Red<RT_RED_MIN> {
  static __device__ __forceinline__ float init() { return INFINITY; }
  static __device__ __forceinline__ float op(float a, float b) { return fminf(a, b); }
};
template <>
struct Red<RT_RED_PROD> {
  static __device__ __forceinline__ float init() { return 1.f; }
  static __device__ __forceinline__ float op(float a, float b) { return a * b; }
};

template <int KIND>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Red<KIND>::op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int KIND>
__device__ __forceinline__ float block_reduce(float v, float* smem) {  // smem: kThreads/32 floats; result valid in all threads
  v = warp_reduce<KIND>(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = Red<KIND>::init();
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) r = Red<KIND>::op(r, smem[i]);
  return r;
}

// ---- inner == 1: warp per row ------------------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(kThreads) row_reduce_warp(const float* __restrict__ x, float* __restrict__ out,
                                                             int64_t rows, int64_t len, float scale) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const float* p = x + r * len;
    float acc = Red<KIND>::init();
    for (int64_t k = lane; k < len; k += 32) acc = Red<KIND>::op(acc, __ldg(p + k));
    acc = warp_reduce<KIND>(acc);
    if (lane == 0) out[r] = acc * scale;
  }
}

// ---- inner == 1, very short rows (class axes, loss tails): one thread per row ---------
// Sums in the association order of the CPU backend's eight-way unrolled fold
// (ndarray sum of a contiguous lane), so that tiny reductions round like the CPU ones.
template <int KIND>
__global__ void __launch_bounds__(kThreads) row_reduce_thread(const float* __restrict__ x, float* __restrict__ out,
                                                               int64_t rows, int len, float scale) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
    const float* p = x + r * len;
    float part[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) part[j] = Red<KIND>::init();
    int k = 0;
    for (; k + 8 <= len; k += 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) part[j] = Red<KIND>::op(part[j], __ldg(p + k + j));
    }
    float acc = Red<KIND>::init();
    acc = Red<KIND>::op(acc, Red<KIND>::op(part[0], part[4]));
    acc = Red<KIND>::op(acc, Red<KIND>::op(part[1], part[5]));
    acc = Red<KIND>::op(acc, Red<KIND>::op(part[2], part[6]));
    acc = Red<KIND>::op(acc, Red<KIND>::op(part[3], part[7]));
    for (; k < len; ++k) acc = Red<KIND>::op(acc, __ldg(p + k));
    out[r] = acc * scale;
  }
}

// ---- inner == 1: block per (row, chunk) --------------------------------------------
// Row r is cut into `chunks` pieces of `chunk_len`; block (r, c) reduces one piece and
// writes out[r * chunks + c].
template <int KIND>
__global__ void __launch_bounds__(kThreads) row_reduce_block(const float* __restrict__ x, float* __restrict__ out,
                                                              int64_t rows, int64_t len, int64_t chunks,
                                                              int64_t chunk_len, float scale) {
  __shared__ float smem[kThreads / 32];
  for (int64_t job = blockIdx.x; job < rows * chunks; job += gridDim.x) {
    int64_t r = job / chunks, c = job % chunks;
    int64_t k0 = c * chunk_len, k1 = k0 + chunk_len;
    if (k1 > len) k1 = len;
    const float* p = x + r * len;
    float acc = Red<KIND>::init();
    // peel to a 16-byte boundary, then 128-bit loads
    int64_t k = k0;
    int64_t mis = ((reinterpret_cast<uintptr_t>(p + k) & 15) >> 2);
    int64_t head = mis ? 4 - mis : 0;
    if (head > k1 - k0) head = k1 - k0;
    if ((int64_t)threadIdx.x < head) acc = Red<KIND>::op(acc, __ldg(p + k + threadIdx.x));
    k += head;
    int64_t n4 = (k1 - k) >> 2;
    const float4* p4 = reinterpret_cast<const float4*>(p + k);
    for (int64_t i = threadIdx.x; i < n4; i += kThreads) {
      float4 v = __ldg(p4 + i);
      acc = Red<KIND>::op(acc, Red<KIND>::op(Red<KIND>::op(v.x, v.y), Red<KIND>::op(v.z, v.w)));
    }
    int64_t t0 = k + (n4 << 2);
    if (t0 + threadIdx.x < k1) acc = Red<KIND>::op(acc, __ldg(p + t0 + threadIdx.x));
    float res = block_reduce<KIND>(acc, smem);
    if (threadIdx.x == 0) out[job] = res * scale;
  }
}

// ---- inner == 1, long rows with 128-bit loads: a warp per row, eight independent loads in flight per lane, no
// block-level synchronisation.
template <int KIND>
__global__ void __launch_bounds__(kThreads) row_reduce_warp_vec(const float* __restrict__ x, float* __restrict__ out,
                                                                 int64_t rows, int len, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n4 = len >> 2;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const float4* p = reinterpret_cast<const float4*>(x + r * len);
    float acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = Red<KIND>::init();
    int k = lane;
    for (; k + 7 * 32 < n4; k += 8 * 32) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(p + k + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        acc[0] = Red<KIND>::op(acc[0], v[u].x);
        acc[1] = Red<KIND>::op(acc[1], v[u].y);
        acc[2] = Red<KIND>::op(acc[2], v[u].z);
        acc[3] = Red<KIND>::op(acc[3], v[u].w);
      }
    }
    for (; k < n4; k += 32) {
      const float4 v = __ldg(p + k);
      acc[0] = Red<KIND>::op(acc[0], v.x);
      acc[1] = Red<KIND>::op(acc[1], v.y);
      acc[2] = Red<KIND>::op(acc[2], v.z);
      acc[3] = Red<KIND>::op(acc[3], v.w);
    }
    float a = Red<KIND>::op(Red<KIND>::op(acc[0], acc[1]), Red<KIND>::op(acc[2], acc[3]));
    a = warp_reduce<KIND>(a);
    if (lane == 0) out[r] = a * scale;
  }
}

// ---- inner == 1, rows of 1024 < len <= 8192 elements: a block per row, the row in registers -------
// Every thread issues all of its 128-bit loads before it uses any of them, so one block keeps
// len*4 bytes in flight; eight resident blocks per SM are enough to cover the HBM latency.
template <int VPT>
__device__ __forceinline__ void load_row_vec(const float* __restrict__ p, int n4, float4 (&v)[VPT], float fill) {
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int k = i * kThreads + threadIdx.x;
    v[i] = k < n4 ? __ldg(reinterpret_cast<const float4*>(p) + k) : make_float4(fill, fill, fill, fill);
  }
}

template <int KIND, int VPT>
__global__ void __launch_bounds__(kThreads) row_reduce_regs(const float* __restrict__ x, float* __restrict__ out,
                                                             int64_t rows, int len, float scale) {
  __shared__ float smem[kThreads / 32];
  const int n4 = len >> 2;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float4 v[VPT];
    load_row_vec<VPT>(x + r * len, n4, v, Red<KIND>::init());
    float acc = Red<KIND>::init();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      acc = Red<KIND>::op(acc, Red<KIND>::op(Red<KIND>::op(v[i].x, v[i].y), Red<KIND>::op(v[i].z, v[i].w)));
    acc = block_reduce<KIND>(acc, smem);
    if (threadIdx.x == 0) out[r] = acc * scale;
  }
}

// ---- inner > 1: column reduction -----------------------------------------------------
// grid: (inner tiles, k-splits, outer); block: (32, 8).  VEC: 4 columns per thread.
template <int KIND, bool VEC, int TX = 32>
__global__ void __launch_bounds__(256) col_reduce(const float* __restrict__ x, float* __restrict__ out, int64_t len,
                                                   int64_t inner, int64_t splits, int64_t rows_per_split, float scale) {
  constexpr int W = VEC ? 4 : 1;
  constexpr int TY = 256 / TX;  // row lanes; a block reads TX*W contiguous columns of TY rows at a time
  __shared__ float red[TY][TX * W + 1];
  int64_t o = blockIdx.z;
  int64_t i0 = ((int64_t)blockIdx.x * TX + threadIdx.x) * W;
  int64_t k0 = (int64_t)blockIdx.y * rows_per_split, k1 = k0 + rows_per_split;
  if (k1 > len) k1 = len;
  float acc[W];
#pragma unroll
  for (int j = 0; j < W; ++j) acc[j] = Red<KIND>::init();
  if (i0 < inner) {
    const float* base = x + o * len * inner + i0;
    int64_t k = k0 + threadIdx.y;
    if (VEC) {
      // four independent 128-bit loads in flight per thread
      for (; k + 3 * TY < k1; k += 4 * TY) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldg(reinterpret_cast<const float4*>(base + (k + TY * u) * inner));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[0] = Red<KIND>::op(acc[0], v[u].x);
          acc[1 % W] = Red<KIND>::op(acc[1 % W], v[u].y);
          acc[2 % W] = Red<KIND>::op(acc[2 % W], v[u].z);
          acc[3 % W] = Red<KIND>::op(acc[3 % W], v[u].w);
        }
      }
    }
    for (; k < k1; k += TY) {
      if (VEC) {
        float4 v = __ldg(reinterpret_cast<const float4*>(base + k * inner));
        acc[0] = Red<KIND>::op(acc[0], v.x);
        acc[1 % W] = Red<KIND>::op(acc[1 % W], v.y);
        acc[2 % W] = Red<KIND>::op(acc[2 % W], v.z);
        acc[3 % W] = Red<KIND>::op(acc[3 % W], v.w);
      } else {
        acc[0] = Red<KIND>::op(acc[0], __ldg(base + k * inner));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < W; ++j) red[threadIdx.y][threadIdx.x * W + j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && i0 < inner) {
#pragma unroll
    for (int j = 0; j < W; ++j) {
      float s = red[0][threadIdx.x * W + j];
#pragma unroll
      for (int y = 1; y < TY; ++y) s = Red<KIND>::op(s, red[y][threadIdx.x * W + j]);
      // out layout [outer, splits, inner]
      out[(o * splits + blockIdx.y) * inner + i0 + j] = s * scale;
    }
  }
}

// ---- inner > 1, split reduction in ONE launch ------------------------------------------------------
// grid: (tiles of 4*TX columns, splits, outer); block: TX column quads x 256/TX row lanes.  Every block writes the partial
// result of its rows; the block that arrives last at its tile's counter (an atomic ticket after a fence) adds the partials
// of all splits in split order - the same order whichever block happens to be last, so the result is reproducible -
// and puts the counter back to zero for the next launch.  Saves the second launch and the pass over its grid.
template <int KIND, int TX>
__global__ void __launch_bounds__(256) col_reduce_single(const float* __restrict__ x, float* __restrict__ part,
                                                          float* __restrict__ out, int64_t len, int64_t inner, int splits,
                                                          int64_t rows_per_split, float scale, unsigned* __restrict__ counters) {
  constexpr int TY = 256 / TX, U = 8;
  __shared__ __align__(16) float red[TY][TX * 4 + 4];
  __shared__ bool last;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  const int64_t o = blockIdx.z;
  const int64_t i0 = ((int64_t)blockIdx.x * TX + tx) * 4;
  const int64_t k0 = (int64_t)blockIdx.y * rows_per_split;
  const int64_t k1 = k0 + rows_per_split < len ? k0 + rows_per_split : len;
  float4 acc = make_float4(Red<KIND>::init(), Red<KIND>::init(), Red<KIND>::init(), Red<KIND>::init());
  auto fold = [&](float4& a, const float4& v) {
    a.x = Red<KIND>::op(a.x, v.x);
    a.y = Red<KIND>::op(a.y, v.y);
    a.z = Red<KIND>::op(a.z, v.z);
    a.w = Red<KIND>::op(a.w, v.w);
  };
  if (i0 < inner) {
    const float* base = x + o * len * inner + i0;
    int64_t k = k0 + ty;
    for (; k + (U - 1) * TY < k1; k += U * TY) {  // eight independent 128-bit loads in flight per thread
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = __ldg(reinterpret_cast<const float4*>(base + (k + TY * u) * inner));
#pragma unroll
      for (int u = 0; u < U; ++u) fold(acc, v[u]);
    }
    for (; k < k1; k += TY) fold(acc, __ldg(reinterpret_cast<const float4*>(base + k * inner)));
  }
  *reinterpret_cast<float4*>(&red[ty][tx * 4]) = acc;
  __syncthreads();
  if (ty == 0 && i0 < inner) {
    float4 r = *reinterpret_cast<const float4*>(&red[0][tx * 4]);
#pragma unroll
    for (int y = 1; y < TY; ++y) fold(r, *reinterpret_cast<const float4*>(&red[y][tx * 4]));
    *reinterpret_cast<float4*>(part + (o * splits + blockIdx.y) * inner + i0) = r;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* counter = counters + o * gridDim.x + blockIdx.x;
    last = atomicAdd(counter, 1u) == (unsigned)splits - 1;
    if (last) *counter = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  acc = make_float4(Red<KIND>::init(), Red<KIND>::init(), Red<KIND>::init(), Red<KIND>::init());
  if (i0 < inner)
    for (int sp = ty; sp < splits; sp += TY) fold(acc, __ldcg(reinterpret_cast<const float4*>(part + (o * splits + sp) * inner + i0)));
  *reinterpret_cast<float4*>(&red[ty][tx * 4]) = acc;
  __syncthreads();
  if (ty == 0 && i0 < inner) {
    float4 r = *reinterpret_cast<const float4*>(&red[0][tx * 4]);
#pragma unroll
    for (int y = 1; y < TY; ++y) fold(r, *reinterpret_cast<const float4*>(&red[y][tx * 4]));
    *reinterpret_cast<float4*>(out + o * inner + i0) = make_float4(r.x * scale, r.y * scale, r.z * scale, r.w * scale);
  }
}

// ---- inner > 1, few rows and a narrow output (a bias gradient, the sum of a few split-K partials of a small matrix) ----------
// One launch of latency-bound size: what counts is that every load is in flight at once.  Block = 32 columns x 32 row lanes; a
// lane takes rows ty, ty + 32, ... with eight independent loads per round; the 32 partial results of a column are combined in
// lane order through shared memory.  grid: (column tiles, outer).
template <int KIND>
__global__ void __launch_bounds__(1024) col_reduce_short(const float* __restrict__ x, float* __restrict__ out, int64_t len, int64_t inner,
                                                          float scale) {
  __shared__ float part[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx, o = blockIdx.y;
  float acc = Red<KIND>::init();
  if (c < inner) {
    const float* base = x + o * len * inner + c;
    int64_t r = ty;
    for (; r + 7 * 32 < len; r += 8 * 32) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(base + (r + 32 * u) * inner);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = Red<KIND>::op(acc, v[u]);
    }
    for (; r < len; r += 32) acc = Red<KIND>::op(acc, __ldg(base + r * inner));
  }
  part[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < inner) {
    float s = part[0][tx];
#pragma unroll
    for (int y = 1; y < 32; ++y) s = Red<KIND>::op(s, part[y][tx]);
    out[o * inner + c] = s * scale;
  }
}

template <int KIND>
rt_status reduce_float(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out, float scale) {
  if (outer * inner == 0) return RT_OK;
  if (len == 0) {  // empty reduction -> identity
    return rt_fill(ctx, out, KIND == RT_RED_SUM ? 0.f : (KIND == RT_RED_PROD ? 1.f : (KIND == RT_RED_MAX ? -INFINITY : INFINITY)),
                   outer * inner);
  }
  const int64_t target_blocks = (int64_t)ctx->sm_count * 4;
  if (inner == 1) {
    int64_t rows = outer;
    if (len <= 16) {
      row_reduce_thread<KIND><<<rt_grid_for(ctx, rows, kThreads), kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, scale);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    if (len <= 1024) {
      int grid = rt_grid_for(ctx, rows, kThreads / 32);
      row_reduce_warp<KIND><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, len, scale);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    if (len > 8192 && len <= 65536 && (len & 3) == 0 && rt_aligned16(x) && rows >= (int64_t)ctx->sm_count * 16) {
      // plenty of very long rows: a warp per row keeps the most loads in flight (up to 8192 elements the block-per-row
      // kernel below, which holds the row in registers, is faster: 12.6 against 14.5 us on 4096 x 4096)
      row_reduce_warp_vec<KIND><<<rt_grid_for(ctx, rows, kThreads / 32), kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, scale);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    if (len <= 8192 && (len & 3) == 0 && rt_aligned16(x) && rows >= 64) {
      const int grid = (int)(rows < (1 << 20) ? rows : (1 << 20));  // a block per row: rows in different phases overlap
      if (len <= 2048) row_reduce_regs<KIND, 2><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, scale);
      else if (len <= 4096) row_reduce_regs<KIND, 4><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, scale);
      else row_reduce_regs<KIND, 8><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, scale);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    int64_t chunks = 1;
    if (rows < target_blocks) {
      chunks = (target_blocks + rows - 1) / rows;
      int64_t max_chunks = (len + 4095) / 4096;  // at least 4096 elements per chunk
      if (chunks > max_chunks) chunks = max_chunks;
      if (chunks < 1) chunks = 1;
    }
    int64_t chunk_len = (len + chunks - 1) / chunks;
    chunk_len = (chunk_len + 3) & ~int64_t(3);
    chunks = (len + chunk_len - 1) / chunk_len;
    int grid = (int)((rows * chunks < target_blocks * 2) ? rows * chunks : target_blocks * 2);
    if (chunks == 1) {
      row_reduce_block<KIND><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, len, 1, chunk_len, scale);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    RtScratch part(ctx);
    rt_status st = part.alloc(sizeof(float) * rows * chunks);
    if (st != RT_OK) return st;
    row_reduce_block<KIND><<<grid, kThreads, 0, ctx->stream>>>(x, part.as<float>(), rows, len, chunks, chunk_len, 1.f);
    RT_LAUNCHED(ctx);
    return reduce_float<KIND>(ctx, part.as<float>(), rows, chunks, 1, out, scale);
  }
  // inner > 1
  bool vec = (inner % 4 == 0) && rt_aligned16(x);
  // wide rows: 2 KB contiguous per row and block (better DRAM page locality than 512 B)
  const bool wide = vec && inner >= 2048;
  const int tile_cols = wide ? 512 : (vec ? 128 : 32);
  int64_t tiles = (inner + tile_cols - 1) / tile_cols;
  int64_t splits = 1;
  // Short reductions (split-K partial sums, bias gradients of a batch) go in one launch: a second pass would cost
  // more than the idle SMs of the first.
  const bool short_reduction = len <= 256 || len * inner <= 65536;
  if (!short_reduction && tiles * outer < target_blocks) {
    splits = (target_blocks + tiles * outer - 1) / (tiles * outer);
    const int min_rows = 64;  // rows per split
    int64_t max_splits = (len + min_rows - 1) / min_rows;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
  }
  if (outer > 65535) {
    // fold very large outer extents through repeated launches
    for (int64_t o0 = 0; o0 < outer; o0 += 65535) {
      int64_t oc = outer - o0 < 65535 ? outer - o0 : 65535;
      rt_status st = reduce_float<KIND>(ctx, x + o0 * len * inner, oc, len, inner, out + o0 * inner, scale);
      if (st != RT_OK) return st;
    }
    return RT_OK;
  }
  if (short_reduction && len >= 16 && outer * inner <= 4096 && outer <= 65535) {
    // few rows, narrow output: one latency-bound launch with all loads in flight (6 us -> 2.5 us for a [256, 10] bias gradient)
    col_reduce_short<KIND><<<dim3((unsigned)((inner + 31) / 32), (unsigned)outer), 1024, 0, ctx->stream>>>(x, out, len, inner, scale);
    RT_LAUNCHED(ctx);
    return RT_OK;
  }
  if (vec && !short_reduction && ctx->reduce_counters) {
    // one launch: 64-column tiles for wide rows (fewer splits, a cheaper finish: 13.9 against 14.4 us on 4096 x 4096), else
    // 128-column tiles; the rows split so that at most four blocks land on every SM (rounded down: a fifth block on some
    // SMs would set the pace)
    const int tile_cols1 = inner >= 2048 ? 64 : 128;
    const int64_t tiles1 = (inner + tile_cols1 - 1) / tile_cols1;
    int64_t sp = 1;
    if (tiles1 * outer < target_blocks) {
      sp = target_blocks / (tiles1 * outer);
      const int64_t max_sp = (len + 63) / 64;
      if (sp > max_sp) sp = max_sp;
      if (sp > 65535) sp = 65535;
    }
    const int64_t rows_per = (len + sp - 1) / sp;
    sp = (len + rows_per - 1) / rows_per;
    if (sp > 1 && tiles1 * outer <= kReduceCounterSlots && tiles1 <= 0x7fffffff) {
      RtScratch partial(ctx);
      rt_status st = partial.alloc(sizeof(float) * outer * sp * inner);
      if (st != RT_OK) return st;
      unsigned* counters = ctx->reduce_counters + (ctx->on_side ? kReduceCounterSlots : 0);
      const dim3 grid1((unsigned)tiles1, (unsigned)sp, (unsigned)outer);
      if (tile_cols1 == 64)
        col_reduce_single<KIND, 16><<<grid1, 256, 0, ctx->stream>>>(x, partial.as<float>(), out, len, inner, (int)sp, rows_per, scale, counters);
      else
        col_reduce_single<KIND, 32><<<grid1, 256, 0, ctx->stream>>>(x, partial.as<float>(), out, len, inner, (int)sp, rows_per, scale, counters);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
  }
  int64_t rps = (len + splits - 1) / splits;
  splits = (len + rps - 1) / rps;
  dim3 grid((unsigned)tiles, (unsigned)splits, (unsigned)outer), block(32, 8);
  RtScratch part(ctx);
  float* dst = out;
  if (splits > 1) {
    rt_status st = part.alloc(sizeof(float) * outer * splits * inner);
    if (st != RT_OK) return st;
    dst = part.as<float>();
  }
  float sc = splits > 1 ? 1.f : scale;
  if (wide) col_reduce<KIND, true, 128><<<grid, dim3(128, 2), 0, ctx->stream>>>(x, dst, len, inner, splits, rps, sc);
  else if (vec) col_reduce<KIND, true><<<grid, block, 0, ctx->stream>>>(x, dst, len, inner, splits, rps, sc);
  else col_reduce<KIND, false><<<grid, block, 0, ctx->stream>>>(x, dst, len, inner, splits, rps, sc);
  RT_LAUNCHED(ctx);
  if (splits > 1) return reduce_float<KIND>(ctx, dst, outer, splits, inner, out, scale);
  return RT_OK;
}

// ---- row-resident softmax-family kernels (inner == 1) ---------------------------------
enum RowMode { ROW_LSE_FWD = 0, ROW_LSE_BWD = 1, ROW_LSM_FWD = 2, ROW_LSM_BWD = 3 };

template <int G>
__device__ __forceinline__ float group_reduce_max(float v, float* smem) {
  if (G == 32) return warp_reduce<RT_RED_MAX>(v);
  return block_reduce<RT_RED_MAX>(v, smem);
}
template <int G>
__device__ __forceinline__ float group_reduce_sum(float v, float* smem) {
  if (G == 32) return warp_reduce<RT_RED_SUM>(v);
  return block_reduce<RT_RED_SUM>(v, smem);
}

// G threads cooperate on one row (G = 32: a warp, several rows per block; G = 256: the block).
// The math follows the reference CPU code: max first, then sum of exp(x - max)
// (src/ops/cpu_ops.rs:462-482, 564-597).  After the first pass the row is re-read from L1/L2.
template <int MODE, int G>
__global__ void __launch_bounds__(kThreads) row_softmax_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                float* __restrict__ out, int64_t rows, int64_t len) {
  __shared__ float smem[kThreads / 32];
  int lane = threadIdx.x % G;
  int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) / G;
  // every thread of a block must take the same number of trips (block_reduce syncs)
  int64_t trips = (rows + ngroups - 1) / ngroups;
  for (int64_t t = 0; t < trips; ++t) {
    int64_t r = group + t * ngroups;
    bool live = r < rows;
    const float* p = x + (live ? r : 0) * len;
    float m = -INFINITY;
    if (live)
      for (int64_t k = lane; k < len; k += G) m = fmaxf(m, __ldg(p + k));
    m = group_reduce_max<G>(m, smem);
    float s = 0.f;
    if (live)
      for (int64_t k = lane; k < len; k += G) s += expf(p[k] - m);
    s = group_reduce_sum<G>(s, smem);
    if (MODE == ROW_LSE_FWD) {
      if (live && lane == 0) out[r] = m + logf(s);
    } else if (MODE == ROW_LSE_BWD) {
      if (live) {
        float lse = m + logf(s), gr = g[r];
        float* o = out + r * len;
        for (int64_t k = lane; k < len; k += G) o[k] = gr * expf(p[k] - lse);
      }
    } else if (MODE == ROW_LSM_FWD) {
      if (live) {
        float ls = logf(s);
        float* o = out + r * len;
        for (int64_t k = lane; k < len; k += G) o[k] = (p[k] - m) - ls;
      }
    } else {  // ROW_LSM_BWD: dx = g - exp(y) * sum(g)
      const float* gp = g + (live ? r : 0) * len;
      float sg = 0.f;
      if (live)
        for (int64_t k = lane; k < len; k += G) sg += __ldg(gp + k);
      sg = group_reduce_sum<G>(sg, smem);
      if (live) {
        float ls = logf(s);
        float* o = out + r * len;
        for (int64_t k = lane; k < len; k += G) o[k] = gp[k] - expf((p[k] - m) - ls) * sg;
      }
    }
  }
}

// Generic strided versions (any inner): one thread per output slice (o, i).
template <int MODE>
__global__ void __launch_bounds__(kThreads) slice_softmax_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                  float* __restrict__ out, int64_t outer, int64_t len,
                                                                  int64_t inner) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < outer * inner; s += stride) {
    int64_t o = s / inner, i = s % inner;
    const float* p = x + o * len * inner + i;
    float m = -INFINITY;
    for (int64_t k = 0; k < len; ++k) m = fmaxf(m, p[k * inner]);
    float sum = 0.f;
    for (int64_t k = 0; k < len; ++k) sum += expf(p[k * inner] - m);
    if (MODE == ROW_LSE_FWD) {
      out[s] = m + logf(sum);
    } else if (MODE == ROW_LSE_BWD) {
      float lse = m + logf(sum), gr = g[s];
      float* q = out + o * len * inner + i;
      for (int64_t k = 0; k < len; ++k) q[k * inner] = gr * expf(p[k * inner] - lse);
    } else if (MODE == ROW_LSM_FWD) {
      float ls = logf(sum);
      float* q = out + o * len * inner + i;
      for (int64_t k = 0; k < len; ++k) q[k * inner] = (p[k * inner] - m) - ls;
    } else {
      const float* gp = g + o * len * inner + i;
      float sg = 0.f;
      for (int64_t k = 0; k < len; ++k) sg += gp[k * inner];
      float ls = logf(sum);
      float* q = out + o * len * inner + i;
      for (int64_t k = 0; k < len; ++k) q[k * inner] = gp[k * inner] - expf((p[k * inner] - m) - ls) * sg;
    }
  }
}

// Rows of 1024 < len <= 8192 elements (len % 4 == 0, 16-byte aligned): a block per row with the row
// (and for log_softmax backward the gradient row) held in registers; global memory is read once and
// written once.  Same formulas as row_softmax_kernel.
template <int MODE, int VPT>
__global__ void __launch_bounds__(kThreads) row_softmax_regs(const float* __restrict__ x, const float* __restrict__ g,
                                                              float* __restrict__ out, int64_t rows, int len) {
  __shared__ float smem[kThreads / 32];
  const int n4 = len >> 2;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float4 v[VPT], gv[VPT];  // gv is used by the log_softmax backward only
    load_row_vec<VPT>(x + r * len, n4, v, -INFINITY);
    if (MODE == ROW_LSM_BWD) load_row_vec<VPT>(g + r * len, n4, gv, 0.f);
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    m = block_reduce<RT_RED_MAX>(m, smem);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)  // padding lanes hold -inf: exp(-inf - m) = 0
      s += (expf(v[i].x - m) + expf(v[i].y - m)) + (expf(v[i].z - m) + expf(v[i].w - m));
    s = block_reduce<RT_RED_SUM>(s, smem);
    if (MODE == ROW_LSE_FWD) {
      if (threadIdx.x == 0) out[r] = m + logf(s);
      continue;
    }
    float4* o = reinterpret_cast<float4*>(out + r * len);
    if (MODE == ROW_LSE_BWD) {
      const float lse = m + logf(s), gr = __ldg(g + r);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = i * kThreads + threadIdx.x;
        if (k < n4) o[k] = make_float4(gr * expf(v[i].x - lse), gr * expf(v[i].y - lse), gr * expf(v[i].z - lse), gr * expf(v[i].w - lse));
      }
    } else if (MODE == ROW_LSM_FWD) {
      const float ls = logf(s);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = i * kThreads + threadIdx.x;
        if (k < n4) o[k] = make_float4((v[i].x - m) - ls, (v[i].y - m) - ls, (v[i].z - m) - ls, (v[i].w - m) - ls);
      }
    } else {  // ROW_LSM_BWD: dx = g - exp(y) * sum(g)
      float sg = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) sg += (gv[i].x + gv[i].y) + (gv[i].z + gv[i].w);
      sg = block_reduce<RT_RED_SUM>(sg, smem);
      const float ls = logf(s);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = i * kThreads + threadIdx.x;
        if (k < n4)
          o[k] = make_float4(gv[i].x - expf((v[i].x - m) - ls) * sg, gv[i].y - expf((v[i].y - m) - ls) * sg,
                             gv[i].z - expf((v[i].z - m) - ls) * sg, gv[i].w - expf((v[i].w - m) - ls) * sg);
      }
    }
  }
}

template <int MODE>
rt_status launch_softmax_family(rt_ctx* ctx, const float* x, const float* g, float* out, int64_t outer, int64_t len,
                                int64_t inner) {
  if (outer * inner == 0) return RT_OK;
  if (inner == 1) {
    if (len <= 1024) {
      int grid = rt_grid_for(ctx, outer, kThreads / 32);
      row_softmax_kernel<MODE, 32><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, len);
    } else if (len <= 8192 && (len & 3) == 0 && rt_aligned16(x) && (MODE == ROW_LSE_FWD || rt_aligned16(out)) &&
               (MODE != ROW_LSM_BWD || rt_aligned16(g))) {
      const int grid = (int)(outer < (1 << 20) ? outer : (1 << 20));  // a block per row: rows in different phases overlap
      if (len <= 2048) row_softmax_regs<MODE, 2><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, (int)len);
      else if (len <= 4096) row_softmax_regs<MODE, 4><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, (int)len);
      else row_softmax_regs<MODE, 8><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, (int)len);
    } else {
      int grid = rt_grid_for(ctx, outer, 1);
      row_softmax_kernel<MODE, kThreads><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, len);
    }
  } else {
    int grid = rt_grid_for(ctx, outer * inner, kThreads);
    slice_softmax_kernel<MODE><<<grid, kThreads, 0, ctx->stream>>>(x, g, out, outer, len, inner);
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// argmax / argmin: one thread per slice, sequential scan (first extremum wins, NaN never wins).
template <bool IS_MAX>
__global__ void __launch_bounds__(kThreads) arg_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t outer,
                                                        int64_t len, int64_t inner) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < outer * inner; s += stride) {
    int64_t o = s / inner, i = s % inner;
    const float* p = x + o * len * inner + i;
    float best = IS_MAX ? -INFINITY : INFINITY;
    int64_t bi = 0;
    for (int64_t k = 0; k < len; ++k) {
      float v = p[k * inner];
      if (IS_MAX ? (v > best) : (v < best)) {
        best = v;
        bi = k;
      }
    }
    out[s] = (float)bi;
  }
}

// dx[o,k,i] = g[o,i] * scale
__global__ void __launch_bounds__(kThreads) expand_axis_kernel(const float* __restrict__ g, float* __restrict__ dx,
                                                                int64_t n, int64_t len, int64_t inner, float scale, bool divide) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t li = len * inner;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    int64_t o = idx / li, i = idx % inner;
    float v = __ldg(g + o * inner + i);
    dx[idx] = divide ? v / scale : v;
  }
}

// dx[:] = g[0] (/ scale): gradient of a global sum / mean
__global__ void __launch_bounds__(kThreads) fill_from_scalar_kernel(const float* __restrict__ g, float* __restrict__ dx,
                                                                     int64_t n, float scale, bool divide) {
  float v = divide ? g[0] / scale : g[0];
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (rt_aligned16(dx)) {
    int64_t n4 = n >> 2;
    float4 v4 = make_float4(v, v, v, v);
    for (int64_t i = tid; i < n4; i += stride) reinterpret_cast<float4*>(dx)[i] = v4;
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) dx[i] = v;
  } else {
    for (int64_t i = tid; i < n; i += stride) dx[i] = v;
  }
}

// ties[o,i] = number of k with |x - ext| < 1e-9   (equal(), src/backend/cpu.rs:715)
__global__ void __launch_bounds__(kThreads) count_ties_kernel(const float* __restrict__ x, const float* __restrict__ ext,
                                                               float* __restrict__ ties, int64_t outer, int64_t len,
                                                               int64_t inner) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < outer * inner; s += stride) {
    int64_t o = s / inner, i = s % inner;
    const float* p = x + o * len * inner + i;
    float e = ext[s], c = 0.f;
    for (int64_t k = 0; k < len; ++k) c += fabsf(p[k * inner] - e) < 1e-9f ? 1.f : 0.f;
    ties[s] = c;
  }
}

// mode 0 (max/min): dx = (g * mask) / (ties + 1e-9);  mode 1 (prod): dx = (g * prod) / (x + 1e-10)
__global__ void __launch_bounds__(kThreads) reduce_bwd_final_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                     const float* __restrict__ r0, const float* __restrict__ r1,
                                                                     float* __restrict__ dx, int64_t n, int64_t len,
                                                                     int64_t inner, int mode) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t li = len * inner;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    int64_t s = (idx / li) * inner + idx % inner;
    float xv = x[idx], gv = g[s];
    if (mode == 0) {
      float mask = fabsf(xv - r0[s]) < 1e-9f ? 1.f : 0.f;
      dx[idx] = (gv * mask) / (r1[s] + 1e-9f);
    } else {
      dx[idx] = (gv * r0[s]) / (xv + 1e-10f);
    }
  }
}

}  // namespace

// out[c] += sum over the rows of x[rows, cols] (rows are few: the bias gradient of one timestep of a recurrent layer, added
// to the gradient the bias already holds).  Block = 32 columns x 8 row lanes: every lane's loads are independent, the eight
// partial sums of a column are added in lane order through shared memory.
__global__ void __launch_bounds__(kThreads) col_sum_accumulate_kernel(const float* __restrict__ x, int64_t rows, int64_t cols,
                                                                       float* __restrict__ out) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  float acc = 0.f;
  if (c < cols) {
    int64_t r = ty;
    for (; r + 24 < rows; r += 32) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldg(x + (r + 8 * u) * cols + c);
      acc += (v[0] + v[1]) + (v[2] + v[3]);
    }
    for (; r < rows; r += 8) acc += __ldg(x + r * cols + c);
  }
  part[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float s = part[0][tx];
#pragma unroll
    for (int y = 1; y < 8; ++y) s += part[y][tx];
    out[c] += s;
  }
}

rt_status rt_sum_axis_internal(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out,
                               float scale) {
  return reduce_float<RT_RED_SUM>(ctx, x, outer, len, inner, out, scale);
}

extern "C" {

rt_status rt_sum_rows_accumulate(rt_ctx* ctx, const float* x, int64_t rows, int64_t cols, float* out) {
  RT_CHECK_CTX(ctx);
  if (rows < 0 || cols < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_sum_rows_accumulate: negative extent");
  if (rows * cols == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, out);
  col_sum_accumulate_kernel<<<(unsigned)((cols + 31) / 32), kThreads, 0, ctx->stream>>>(x, rows, cols, out);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_reduce(rt_ctx* ctx, int kind, const float* x, int64_t outer, int64_t len, int64_t inner, float* out) {
  RT_CHECK_CTX(ctx);
  if (kind < 0 || kind >= RT_RED_COUNT) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_reduce: unknown kind %d", kind);
  if (outer < 0 || len < 0 || inner < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_reduce: negative extent");
  if (outer * inner == 0) return RT_OK;
  RT_CHECK_PTR(ctx, out);
  if (len > 0) RT_CHECK_PTR(ctx, x);
  switch (kind) {
    case RT_RED_SUM: return reduce_float<RT_RED_SUM>(ctx, x, outer, len, inner, out, 1.f);
    case RT_RED_MEAN: {
      if (len == 0) RT_FAIL(ctx, RT_ERR_EMPTY_TENSOR, "mean over an empty axis");
      // the CPU backend divides the sum by n (ndarray mean_axis): scale by a reciprocal would round differently
      rt_status st = reduce_float<RT_RED_SUM>(ctx, x, outer, len, inner, out, 1.f);
      if (st != RT_OK) return st;
      return rt_unary(ctx, RT_DIV_SCALAR, out, out, outer * inner, (float)len, 0.f);
    }
    case RT_RED_MAX: return reduce_float<RT_RED_MAX>(ctx, x, outer, len, inner, out, 1.f);
    case RT_RED_MIN: return reduce_float<RT_RED_MIN>(ctx, x, outer, len, inner, out, 1.f);
    case RT_RED_PROD: return reduce_float<RT_RED_PROD>(ctx, x, outer, len, inner, out, 1.f);
    case RT_RED_LOGSUMEXP: return launch_softmax_family<ROW_LSE_FWD>(ctx, x, nullptr, out, outer, len, inner);
    case RT_RED_ARGMAX:
      arg_kernel<true><<<rt_grid_for(ctx, outer * inner, kThreads), kThreads, 0, ctx->stream>>>(x, out, outer, len, inner);
      RT_LAUNCHED(ctx);
      return RT_OK;
    case RT_RED_ARGMIN:
      arg_kernel<false><<<rt_grid_for(ctx, outer * inner, kThreads), kThreads, 0, ctx->stream>>>(x, out, outer, len, inner);
      RT_LAUNCHED(ctx);
      return RT_OK;
  }
  return RT_ERR_INTERNAL;
}

rt_status rt_reduce_backward(rt_ctx* ctx, int kind, const float* x, const float* g, int64_t outer, int64_t len,
                             int64_t inner, float* dx) {
  RT_CHECK_CTX(ctx);
  if (outer < 0 || len < 0 || inner < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_reduce_backward: negative extent");
  int64_t n = outer * len * inner;
  if (n == 0) return RT_OK;
  RT_CHECK_PTR(ctx, g);
  RT_CHECK_PTR(ctx, dx);
  int grid = rt_grid_for(ctx, n, kThreads * 2);
  switch (kind) {
    case RT_RED_SUM:
      if (outer * inner == 1) fill_from_scalar_kernel<<<rt_grid_for(ctx, (n + 3) / 4, kThreads * 2), kThreads, 0, ctx->stream>>>(g, dx, n, 1.f, false);
      else expand_axis_kernel<<<grid, kThreads, 0, ctx->stream>>>(g, dx, n, len, inner, 1.f, false);
      RT_LAUNCHED(ctx);
      return RT_OK;
    case RT_RED_MEAN:  // div_scalar(broadcast(g), len)  (src/ops/cpu_backward.rs:716,764)
      if (outer * inner == 1) fill_from_scalar_kernel<<<rt_grid_for(ctx, (n + 3) / 4, kThreads * 2), kThreads, 0, ctx->stream>>>(g, dx, n, (float)len, true);
      else expand_axis_kernel<<<grid, kThreads, 0, ctx->stream>>>(g, dx, n, len, inner, (float)len, true);
      RT_LAUNCHED(ctx);
      return RT_OK;
    case RT_RED_MAX:
    case RT_RED_MIN: {
      RT_CHECK_PTR(ctx, x);
      RtScratch ext(ctx), ties(ctx);
      rt_status st = ext.alloc(sizeof(float) * outer * inner);
      if (st == RT_OK) st = ties.alloc(sizeof(float) * outer * inner);
      if (st != RT_OK) return st;
      st = rt_reduce(ctx, kind, x, outer, len, inner, ext.as<float>());
      if (st != RT_OK) return st;
      count_ties_kernel<<<rt_grid_for(ctx, outer * inner, kThreads), kThreads, 0, ctx->stream>>>(x, ext.as<float>(), ties.as<float>(), outer, len, inner);
      RT_LAUNCHED(ctx);
      reduce_bwd_final_kernel<<<grid, kThreads, 0, ctx->stream>>>(x, g, ext.as<float>(), ties.as<float>(), dx, n, len, inner, 0);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    case RT_RED_PROD: {
      RT_CHECK_PTR(ctx, x);
      RtScratch pr(ctx);
      rt_status st = pr.alloc(sizeof(float) * outer * inner);
      if (st != RT_OK) return st;
      st = rt_reduce(ctx, RT_RED_PROD, x, outer, len, inner, pr.as<float>());
      if (st != RT_OK) return st;
      reduce_bwd_final_kernel<<<grid, kThreads, 0, ctx->stream>>>(x, g, pr.as<float>(), nullptr, dx, n, len, inner, 1);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    case RT_RED_LOGSUMEXP:
      RT_CHECK_PTR(ctx, x);
      return launch_softmax_family<ROW_LSE_BWD>(ctx, x, g, dx, outer, len, inner);
    default:
      RT_FAIL(ctx, RT_ERR_UNIMPLEMENTED, "rt_reduce_backward: kind %d has no gradient", kind);
  }
}

rt_status rt_sum_all_host(rt_ctx* ctx, const float* x, int64_t n, float* host_out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, host_out);
  if (n == 0) {
    *host_out = 0.f;
    return RT_OK;
  }
  RtScratch s(ctx);
  rt_status st = s.alloc(sizeof(float));
  if (st != RT_OK) return st;
  st = reduce_float<RT_RED_SUM>(ctx, x, 1, n, 1, s.as<float>(), 1.f);
  if (st != RT_OK) return st;
  return rt_memcpy_d2h(ctx, host_out, s.ptr, sizeof(float));
}

rt_status rt_log_softmax(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* y) {
  RT_CHECK_CTX(ctx);
  if (outer * len * inner == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, y);
  return launch_softmax_family<ROW_LSM_FWD>(ctx, x, nullptr, y, outer, len, inner);
}

rt_status rt_log_softmax_backward(rt_ctx* ctx, const float* x, const float* g, int64_t outer, int64_t len, int64_t inner,
                                  float* dx) {
  RT_CHECK_CTX(ctx);
  if (outer * len * inner == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, g);
  RT_CHECK_PTR(ctx, dx);
  return launch_softmax_family<ROW_LSM_BWD>(ctx, x, g, dx, outer, len, inner);
}

}  // extern "C"

// ---- axis sum whose workspace is a fixed array in device memory --------------------------------
// Some callers may not touch the allocator at all while they enqueue work: a stream that is being
// captured into a graph (an allocation made during capture belongs to no replay), or a host loop
// that promised its latency budget no driver call that can block.  For them the split partial sums
// of the axis reduction live in the array below instead of a block from the context's allocator.
// The array exists once per device (it is part of the loaded module), so two calls that overlap on
// one device - different streams, different contexts, or a graph replay next to an eager call -
// would write each other's partial sums; calls on one stream are ordered and safe.  It keeps
// whatever the previous call left in it: the first pass writes every slot the second pass reads,
// so nothing has to start at zero and nothing is cleared.
namespace {

constexpr int64_t kStaticScratchFloats = int64_t(1) << 18;  // 1 MiB of partial sums
__device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Address of the array on the context's device, looked up once per device with that device current.
// The first lookup may make the runtime load the module, so it belongs before any stream capture.
rt_status static_scratch(rt_ctx* ctx, float** out) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_reduce_sum_static_scratch: device ordinal %d out of range", ctx->device);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[ctx->device]) {
    int current = -1;
    RT_CUDA(ctx, cudaGetDevice(&current));
    if (current != ctx->device) RT_CUDA(ctx, cudaSetDevice(ctx->device));
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (current != ctx->device) cudaSetDevice(current);
    if (e != cudaSuccess || !p)
      RT_FAIL(ctx, RT_ERR_CUDA, "rt_reduce_sum_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_scratch_ptr[ctx->device] = p;
  }
  *out = g_static_scratch_ptr[ctx->device];
  return RT_OK;
}

}  // namespace

extern "C" rt_status rt_reduce_sum_static_scratch(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner,
                                                  float* out) {
  RT_CHECK_CTX(ctx);
  if (outer < 0 || len < 0 || inner < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_reduce_sum_static_scratch: negative extent");
  float* scratch = nullptr;
  rt_status st = static_scratch(ctx, &scratch);  // also serves as the set-up call
  if (st != RT_OK) return st;
  if (outer * inner == 0) return RT_OK;
  RT_CHECK_PTR(ctx, out);
  if (len == 0) return rt_fill(ctx, out, 0.f, outer * inner);
  RT_CHECK_PTR(ctx, x);
  if (outer > 65535 && inner > 1)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_reduce_sum_static_scratch: outer extent %lld exceeds 65535", (long long)outer);
  const int64_t target_blocks = (int64_t)ctx->sm_count * 4;
  if (inner == 1) {
    const int64_t rows = outer;
    if (len <= 16) {
      row_reduce_thread<RT_RED_SUM><<<rt_grid_for(ctx, rows, kThreads), kThreads, 0, ctx->stream>>>(x, out, rows, (int)len, 1.f);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    if (len <= 1024) {
      row_reduce_warp<RT_RED_SUM><<<rt_grid_for(ctx, rows, kThreads / 32), kThreads, 0, ctx->stream>>>(x, out, rows, len, 1.f);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    // long rows: cut each into chunks of at least 4096 elements, one partial sum per chunk
    int64_t chunks = 1;
    if (rows < target_blocks) {
      chunks = (target_blocks + rows - 1) / rows;
      const int64_t max_chunks = (len + 4095) / 4096;
      if (chunks > max_chunks) chunks = max_chunks;
      if (chunks > 1024) chunks = 1024;  // the second pass is one warp per row
      if (chunks < 1) chunks = 1;
    }
    int64_t chunk_len = (len + chunks - 1) / chunks;
    chunk_len = (chunk_len + 3) & ~int64_t(3);
    chunks = (len + chunk_len - 1) / chunk_len;
    const int grid = (int)((rows * chunks < target_blocks * 2) ? rows * chunks : target_blocks * 2);
    if (chunks == 1) {
      row_reduce_block<RT_RED_SUM><<<grid, kThreads, 0, ctx->stream>>>(x, out, rows, len, 1, chunk_len, 1.f);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    if (rows * chunks > kStaticScratchFloats)
      RT_FAIL(ctx, RT_ERR_INVALID_OPERATION,
              "rt_reduce_sum_static_scratch: %lld partial sums needed, the fixed workspace holds %lld", (long long)(rows * chunks),
              (long long)kStaticScratchFloats);
    row_reduce_block<RT_RED_SUM><<<grid, kThreads, 0, ctx->stream>>>(x, scratch, rows, len, chunks, chunk_len, 1.f);
    RT_LAUNCHED(ctx);
    if (chunks <= 16)
      row_reduce_thread<RT_RED_SUM><<<rt_grid_for(ctx, rows, kThreads), kThreads, 0, ctx->stream>>>(scratch, out, rows, (int)chunks, 1.f);
    else
      row_reduce_warp<RT_RED_SUM><<<rt_grid_for(ctx, rows, kThreads / 32), kThreads, 0, ctx->stream>>>(scratch, out, rows, chunks, 1.f);
    RT_LAUNCHED(ctx);
    return RT_OK;
  }
  // inner > 1: column sums, the reduced axis cut into splits of at least 64 rows
  const bool vec = (inner % 4 == 0) && rt_aligned16(x);
  const int64_t tiles = (inner + (vec ? 128 : 32) - 1) / (vec ? 128 : 32);
  int64_t splits = 1;
  if (tiles * outer < target_blocks) {
    splits = (target_blocks + tiles * outer - 1) / (tiles * outer);
    const int64_t max_splits = (len + 63) / 64;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
  }
  const int64_t rps = (len + splits - 1) / splits;
  splits = (len + rps - 1) / rps;
  if (splits > 1 && outer * splits * inner > kStaticScratchFloats)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION,
            "rt_reduce_sum_static_scratch: %lld partial sums needed, the fixed workspace holds %lld",
            (long long)(outer * splits * inner), (long long)kStaticScratchFloats);
  dim3 grid((unsigned)tiles, (unsigned)splits, (unsigned)outer), block(32, 8);
  float* dst = splits > 1 ? scratch : out;
  if (vec) col_reduce<RT_RED_SUM, true><<<grid, block, 0, ctx->stream>>>(x, dst, len, inner, splits, rps, 1.f);
  else col_reduce<RT_RED_SUM, false><<<grid, block, 0, ctx->stream>>>(x, dst, len, inner, splits, rps, 1.f);
  RT_LAUNCHED(ctx);
  if (splits > 1) {
    // second pass in one launch: the partial sums [outer, splits, inner] are 256-byte aligned, inner % 4 decides the width
    const bool vec2 = inner % 4 == 0;
    dim3 grid2((unsigned)((inner + (vec2 ? 128 : 32) - 1) / (vec2 ? 128 : 32)), 1, (unsigned)outer);
    if (vec2) col_reduce<RT_RED_SUM, true><<<grid2, block, 0, ctx->stream>>>(scratch, out, splits, inner, 1, splits, 1.f);
    else col_reduce<RT_RED_SUM, false><<<grid2, block, 0, ctx->stream>>>(scratch, out, splits, inner, 1, splits, 1.f);
    RT_LAUNCHED(ctx);
  }
  return RT_OK;
}

// ---- fused classification loss ---------------------------------------------------------------------------------------
// loss = -(1/rows) * sum_b sum_k targets[b,k] * log_softmax(logits)[b,k]: the chain log_softmax -> mul -> sum(axis 1) ->
// mean -> mul(-1) of the reference's training examples (examples/train_mnist_cpu.rs:63-97) in one kernel forward and
// one backward.  No counterpart in the reference.  One thread per row (classification heads have tens of classes);
// the row losses are added by one block in a fixed order.
namespace {

__device__ __forceinline__ void row_max_lse(const float* __restrict__ x, int classes, float& m, float& lse) {
  m = -INFINITY;
  for (int k = 0; k < classes; ++k) m = fmaxf(m, __ldg(x + k));
  float s = 0.f;
  for (int k = 0; k < classes; ++k) s += expf(__ldg(x + k) - m);
  lse = logf(s);
}

__global__ void __launch_bounds__(kThreads) sce_forward_kernel(const float* __restrict__ logits, const float* __restrict__ targets,
                                                               float* __restrict__ loss, int64_t rows, int classes) {
  __shared__ float smem[kThreads / 32];
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < rows; r += kThreads) {
    const float* x = logits + r * classes;
    const float* t = targets + r * classes;
    float m, lse;
    row_max_lse(x, classes, m, lse);
    float e = 0.f;
    for (int k = 0; k < classes; ++k) e += ((__ldg(x + k) - m) - lse) * __ldg(t + k);
    acc += e;
  }
  acc = block_reduce<RT_RED_SUM>(acc, smem);
  if (threadIdx.x == 0) loss[0] = (acc / (float)rows) * -1.0f;
}

// dlogits = -(g/rows) * (t - softmax * sum_k t);  dtargets (optional) = -(g/rows) * log_softmax
__global__ void __launch_bounds__(kThreads) sce_backward_kernel(const float* __restrict__ logits, const float* __restrict__ targets,
                                                                const float* __restrict__ g, float* __restrict__ dlogits,
                                                                float* __restrict__ dtargets, int64_t rows, int classes) {
  const float scale = -__ldg(g) / (float)rows;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    const float* x = logits + r * classes;
    const float* t = targets + r * classes;
    float m, lse;
    row_max_lse(x, classes, m, lse);
    float st = 0.f;
    for (int k = 0; k < classes; ++k) st += __ldg(t + k) * scale;  // sum of the upstream gradient of log_softmax
    for (int k = 0; k < classes; ++k) {
      const float ls = (__ldg(x + k) - m) - lse;
      if (dlogits) dlogits[r * classes + k] = __ldg(t + k) * scale - expf(ls) * st;
      if (dtargets) dtargets[r * classes + k] = ls * scale;
    }
  }
}

// ---- the same two kernels with a warp per row (lanes over the classes, coalesced), used for more than 16 classes ----
__device__ __forceinline__ float warp_sum_all(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_all(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void row_max_lse_warp(const float* x, int classes, int lane, float& m, float& lse) {
  float mm = -INFINITY;
  for (int k = lane; k < classes; k += 32) mm = fmaxf(mm, __ldg(x + k));
  m = warp_max_all(mm);
  float ss = 0.f;
  for (int k = lane; k < classes; k += 32) ss += expf(__ldg(x + k) - m);
  lse = logf(warp_sum_all(ss));
}

constexpr int kSceWarpBlock = 1024;
// part[block] = sum over the block's rows of sum_k log_softmax * t; with `final` the single block writes the loss itself.
__global__ void __launch_bounds__(kSceWarpBlock) sce_forward_warp_kernel(const float* __restrict__ logits,
                                                                         const float* __restrict__ targets, float* __restrict__ out,
                                                                         int64_t rows, int classes, int final) {
  __shared__ float smem[kSceWarpBlock / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int nw = kSceWarpBlock / 32;
  float acc = 0.f;
  for (int64_t r = (int64_t)blockIdx.x * nw + warp; r < rows; r += (int64_t)gridDim.x * nw) {
    const float* x = logits + r * classes;
    const float* t = targets + r * classes;
    float m, lse;
    row_max_lse_warp(x, classes, lane, m, lse);
    float e = 0.f;
    for (int k = lane; k < classes; k += 32) e += ((__ldg(x + k) - m) - lse) * __ldg(t + k);
    acc += warp_sum_all(e);
  }
  if (lane == 0) smem[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < nw; ++w) total += smem[w];
    out[blockIdx.x] = final ? (total / (float)rows) * -1.0f : total;
  }
}

__global__ void __launch_bounds__(32) sce_finish_kernel(const float* __restrict__ part, int n, float* __restrict__ loss, int64_t rows) {
  float v = 0.f;
  for (int i = threadIdx.x; i < n; i += 32) v += part[i];
  v = warp_sum_all(v);
  if (threadIdx.x == 0) loss[0] = (v / (float)rows) * -1.0f;
}

__global__ void __launch_bounds__(kThreads) sce_backward_warp_kernel(const float* __restrict__ logits, const float* __restrict__ targets,
                                                                     const float* __restrict__ g, float* __restrict__ dlogits,
                                                                     float* __restrict__ dtargets, int64_t rows, int classes) {
  const float scale = -__ldg(g) / (float)rows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int nw = kThreads / 32;
  for (int64_t r = (int64_t)blockIdx.x * nw + warp; r < rows; r += (int64_t)gridDim.x * nw) {
    const float* x = logits + r * classes;
    const float* t = targets + r * classes;
    float m, lse;
    row_max_lse_warp(x, classes, lane, m, lse);
    float st = 0.f;
    for (int k = lane; k < classes; k += 32) st += __ldg(t + k) * scale;
    st = warp_sum_all(st);
    for (int k = lane; k < classes; k += 32) {
      const float ls = (__ldg(x + k) - m) - lse;
      if (dlogits) dlogits[r * classes + k] = __ldg(t + k) * scale - expf(ls) * st;
      if (dtargets) dtargets[r * classes + k] = ls * scale;
    }
  }
}

}  // namespace

extern "C" rt_status rt_softmax_cross_entropy(rt_ctx* ctx, const float* logits, const float* targets, int64_t rows, int64_t classes,
                                              float* loss) {
  RT_CHECK_CTX(ctx);
  if (rows <= 0 || classes <= 0) RT_FAIL(ctx, RT_ERR_EMPTY_TENSOR, "rt_softmax_cross_entropy: empty input");
  if (classes > 4096 || rows > (int64_t(1) << 24))
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_softmax_cross_entropy: at most 4096 classes and 2^24 rows");
  RT_CHECK_PTR(ctx, logits);
  RT_CHECK_PTR(ctx, targets);
  RT_CHECK_PTR(ctx, loss);
  if (classes <= 16) {  // a thread per row
    sce_forward_kernel<<<1, kThreads, 0, ctx->stream>>>(logits, targets, loss, rows, (int)classes);
    RT_LAUNCHED(ctx);
    return RT_OK;
  }
  constexpr int rows_per_block = kSceWarpBlock / 32;
  if (rows <= 8 * rows_per_block) {
    sce_forward_warp_kernel<<<1, kSceWarpBlock, 0, ctx->stream>>>(logits, targets, loss, rows, (int)classes, 1);
    RT_LAUNCHED(ctx);
    return RT_OK;
  }
  int64_t want = (rows + 4 * rows_per_block - 1) / (4 * rows_per_block);
  const int grid = (int)(want < ctx->sm_count ? want : ctx->sm_count);
  RtScratch part(ctx);
  rt_status st = part.alloc(sizeof(float) * (size_t)grid);
  if (st != RT_OK) return st;
  sce_forward_warp_kernel<<<grid, kSceWarpBlock, 0, ctx->stream>>>(logits, targets, part.as<float>(), rows, (int)classes, 0);
  RT_LAUNCHED(ctx);
  sce_finish_kernel<<<1, 32, 0, ctx->stream>>>(part.as<float>(), grid, loss, rows);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

extern "C" rt_status rt_softmax_cross_entropy_backward(rt_ctx* ctx, const float* logits, const float* targets, const float* g,
                                                       int64_t rows, int64_t classes, float* dlogits, float* dtargets) {
  RT_CHECK_CTX(ctx);
  if (rows <= 0 || classes <= 0) return RT_OK;
  if (classes > 4096) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_softmax_cross_entropy_backward: at most 4096 classes");
  RT_CHECK_PTR(ctx, logits);
  RT_CHECK_PTR(ctx, targets);
  RT_CHECK_PTR(ctx, g);
  if (!dlogits && !dtargets) return RT_OK;
  if (classes <= 16)
    sce_backward_kernel<<<rt_grid_for(ctx, rows, kThreads), kThreads, 0, ctx->stream>>>(logits, targets, g, dlogits, dtargets, rows,
                                                                                       (int)classes);
  else
    sce_backward_warp_kernel<<<rt_grid_for(ctx, rows, kThreads / 32), kThreads, 0, ctx->stream>>>(logits, targets, g, dlogits,
                                                                                                 dtargets, rows, (int)classes);
  RT_LAUNCHED(ctx);
  return RT_OK;
}
