// Elementwise forward / backward kernels with fused un-broadcast reductions,
// plus the layout helpers (broadcast_to, transpose, slice, slice_assign, fill).
//
// All kernels are HBM-bandwidth bound: 128-bit loads/stores when the pointers are
// 16-byte aligned, grid-stride loops on a grid capped at a few waves of the SM count.
#include <cmath>

#include "rt_internal.cuh"

namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------
// unary functors: y = f(x);  dx = g * f'(x) with f' recomputed from x, in the same
// algebraic form as the reference CPU backend (src/backend/cpu.rs) so that results
// agree to rounding.
// ---------------------------------------------------------------------------------
template <int OP>
struct Unary;
#define RT_DEF_UNARY(OPC, FWD, BWD)                                                      \
  template <>                                                                            \
  struct Unary<OPC> {                                                                    \
    static __device__ __forceinline__ float fwd(float x, float p0, float p1) { return FWD; } \
    static __device__ __forceinline__ float bwd(float x, float g, float p0, float p1) { return BWD; } \
  };
RT_DEF_UNARY(RT_RELU, fmaxf(x, 0.f), g * (x > 0.f ? 1.f : 0.f))                            // cpu_backward.rs:783-798
RT_DEF_UNARY(RT_ELU, (x < 0.f ? p0 * (expf(x) - 1.f) : x), g * (x < 0.f ? p0 * expf(x) : 1.f))  // cpu.rs:1345,1525
RT_DEF_UNARY(RT_EXP, expf(x), g * expf(x))                                                 // cpu.rs:1634-1646
RT_DEF_UNARY(RT_LN, logf(x), g * (1.f / x))                                                // cpu.rs:1648-1661
RT_DEF_UNARY(RT_SIN, sinf(x), cosf(x) * g)                                                 // cpu.rs:2089-2115
RT_DEF_UNARY(RT_COS, cosf(x), -sinf(x) * g)                                                // cpu.rs:2133-2159
RT_DEF_UNARY(RT_TAN, tanf(x), g * (1.f / (cosf(x) * cosf(x))))                             // cpu.rs:2177-2202
RT_DEF_UNARY(RT_SQUARE, x * x, g * (2.f * x))                                              // cpu.rs:1793-1815
RT_DEF_UNARY(RT_SQRT, sqrtf(x), g * (0.5f / sqrtf(x)))                                     // cpu.rs:1725-1735
RT_DEF_UNARY(RT_ABS, fabsf(x), g * (x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f)))               // cpu.rs:1667-1687
RT_DEF_UNARY(RT_CLIP, fminf(fmaxf(x, p0), p1), g * ((x >= p0 && x <= p1) ? 1.f : 0.f))     // cpu.rs:2385-2413
RT_DEF_UNARY(RT_MUL_SCALAR, x * p0, g * p0)                                                // ops/mod.rs:801-824
RT_DEF_UNARY(RT_DIV_SCALAR, x / p0, g / p0)                                                // cpu.rs:1271-1279
RT_DEF_UNARY(RT_SOFTPLUS, logf(1.f + expf(x)), g * (1.f / (1.f + expf(-x))))               // cpu.rs:1737-1762
#undef RT_DEF_UNARY
template <>
struct Unary<RT_TANH> {  // cpu.rs:1372-1394: g * (1 - tanh(x)^2)
  static __device__ __forceinline__ float fwd(float x, float, float) { return tanhf(x); }
  static __device__ __forceinline__ float bwd(float x, float g, float, float) {
    float y = tanhf(x);
    return g * (1.f - y * y);
  }
};
template <>
struct Unary<RT_SIGMOID> {  // cpu.rs:1693-1715: g * (y * (1 - y))
  static __device__ __forceinline__ float fwd(float x, float, float) { return 1.f / (1.f + expf(-x)); }
  static __device__ __forceinline__ float bwd(float x, float g, float, float) {
    float y = 1.f / (1.f + expf(-x));
    return g * (y * (1.f - y));
  }
};

template <int OP, bool VEC>
__global__ void __launch_bounds__(kThreads) unary_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                              int64_t n, float p0, float p1) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = __ldg(x4 + i);
      v.x = Unary<OP>::fwd(v.x, p0, p1);
      v.y = Unary<OP>::fwd(v.y, p0, p1);
      v.z = Unary<OP>::fwd(v.z, p0, p1);
      v.w = Unary<OP>::fwd(v.w, p0, p1);
      y4[i] = v;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) y[i] = Unary<OP>::fwd(x[i], p0, p1);
  } else {
    for (int64_t i = tid; i < n; i += stride) y[i] = Unary<OP>::fwd(x[i], p0, p1);
  }
}

template <int OP, bool VEC>
__global__ void __launch_bounds__(kThreads) unary_bwd_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                              float* __restrict__ dx, int64_t n, float p0, float p1) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* g4 = reinterpret_cast<const float4*>(g);
    float4* d4 = reinterpret_cast<float4*>(dx);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = __ldg(x4 + i), gg = __ldg(g4 + i), r;
      r.x = Unary<OP>::bwd(v.x, gg.x, p0, p1);
      r.y = Unary<OP>::bwd(v.y, gg.y, p0, p1);
      r.z = Unary<OP>::bwd(v.z, gg.z, p0, p1);
      r.w = Unary<OP>::bwd(v.w, gg.w, p0, p1);
      d4[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) dx[i] = Unary<OP>::bwd(x[i], g[i], p0, p1);
  } else {
    for (int64_t i = tid; i < n; i += stride) dx[i] = Unary<OP>::bwd(x[i], g[i], p0, p1);
  }
}

template <int OP>
void launch_unary_fwd(rt_ctx* ctx, const float* x, float* y, int64_t n, float p0, float p1) {
  bool vec = rt_aligned16(x) && rt_aligned16(y);
  int grid = rt_grid_for(ctx, vec ? (n + 3) / 4 : n, kThreads * 2);
  if (vec) unary_fwd_kernel<OP, true><<<grid, kThreads, 0, ctx->stream>>>(x, y, n, p0, p1);
  else unary_fwd_kernel<OP, false><<<grid, kThreads, 0, ctx->stream>>>(x, y, n, p0, p1);
}
template <int OP>
void launch_unary_bwd(rt_ctx* ctx, const float* x, const float* g, float* dx, int64_t n, float p0, float p1) {
  bool vec = rt_aligned16(x) && rt_aligned16(g) && rt_aligned16(dx);
  int grid = rt_grid_for(ctx, vec ? (n + 3) / 4 : n, kThreads * 2);
  if (vec) unary_bwd_kernel<OP, true><<<grid, kThreads, 0, ctx->stream>>>(x, g, dx, n, p0, p1);
  else unary_bwd_kernel<OP, false><<<grid, kThreads, 0, ctx->stream>>>(x, g, dx, n, p0, p1);
}

// ---------------------------------------------------------------------------------
// binary functors
// ---------------------------------------------------------------------------------
template <int OP>
struct Binary;
#define RT_DEF_BINARY(OPC, FWD, DA, DB)                                                   \
  template <>                                                                             \
  struct Binary<OPC> {                                                                    \
    static __device__ __forceinline__ float fwd(float a, float b) { return FWD; }         \
    static __device__ __forceinline__ float da(float a, float b, float g) { return DA; }  \
    static __device__ __forceinline__ float db(float a, float b, float g) { return DB; }  \
  };
RT_DEF_BINARY(RT_ADD, a + b, g, g)                                                  // cpu_backward.rs:163-184
RT_DEF_BINARY(RT_SUB, a - b, g, g / -1.f)                                           // cpu.rs:1617-1632
RT_DEF_BINARY(RT_MUL, a * b, g * b, g * a)                                          // cpu_backward.rs:136-160
RT_DEF_BINARY(RT_DIV, a / b, g * (1.f / b), g * ((a / (b * b)) / -1.f))             // cpu.rs:1592-1615
RT_DEF_BINARY(RT_POWF, powf(a, b), g * (b * powf(a, b - 1.f)), g * (powf(a, b) * logf(a)))  // cpu_backward.rs:467-520
RT_DEF_BINARY(RT_MAXIMUM, fmaxf(a, b), g * (a >= b ? 1.f : 0.f), g * (b > a ? 1.f : 0.f))   // cpu.rs:1865-1942
RT_DEF_BINARY(RT_MINIMUM, fminf(a, b), g * (a <= b ? 1.f : 0.f), g * (b < a ? 1.f : 0.f))   // cpu.rs:1992-2071
RT_DEF_BINARY(RT_EQUAL, (fabsf(a - b) < 1e-9f ? 1.f : 0.f), 0.f, 0.f)               // cpu.rs:684-722
RT_DEF_BINARY(RT_NOT_EQUAL, (fabsf(a - b) >= 1e-9f ? 1.f : 0.f), 0.f, 0.f)          // cpu.rs:860-898
RT_DEF_BINARY(RT_GREATER, (a > b ? 1.f : 0.f), 0.f, 0.f)
RT_DEF_BINARY(RT_GREATER_EQUAL, (a >= b ? 1.f : 0.f), 0.f, 0.f)
RT_DEF_BINARY(RT_LESS, (a < b ? 1.f : 0.f), 0.f, 0.f)
RT_DEF_BINARY(RT_LESS_EQUAL, (a <= b ? 1.f : 0.f), 0.f, 0.f)
#undef RT_DEF_BINARY

// Collapsed broadcast geometry: out dims (outermost first) with element strides of
// a and b (0 where broadcast).
struct BcastGeom {
  int nd;
  int64_t shape[RT_MAX_DIMS];
  int64_t sa[RT_MAX_DIMS];
  int64_t sb[RT_MAX_DIMS];
  int64_t numel;
};

// mode 0: a[i], b[i]   mode 1: a[i], b[0]   mode 2: a[0], b[i]
// mode 3: a[i], b[i % cols]   mode 4: a[i % cols], b[i]
template <int OP, int MODE, bool VEC>
__global__ void __launch_bounds__(kThreads) binary_fwd_fast(const float* __restrict__ a, const float* __restrict__ b,
                                                             float* __restrict__ out, int64_t n, int64_t cols) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  auto la = [&](int64_t i) { return MODE == 2 ? a[0] : (MODE == 4 ? __ldg(a + i % cols) : a[i]); };
  auto lb = [&](int64_t i) { return MODE == 1 ? b[0] : (MODE == 3 ? __ldg(b + i % cols) : b[i]); };
  if (VEC) {  // cols % 4 == 0 in modes 3/4, so a float4 never straddles a row
    int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 va, vb, r;
      if (MODE == 2) { float s = a[0]; va = make_float4(s, s, s, s); }
      else if (MODE == 4) va = __ldg(reinterpret_cast<const float4*>(a) + (i % (cols >> 2)));
      else va = __ldg(reinterpret_cast<const float4*>(a) + i);
      if (MODE == 1) { float s = b[0]; vb = make_float4(s, s, s, s); }
      else if (MODE == 3) vb = __ldg(reinterpret_cast<const float4*>(b) + (i % (cols >> 2)));
      else vb = __ldg(reinterpret_cast<const float4*>(b) + i);
      r.x = Binary<OP>::fwd(va.x, vb.x);
      r.y = Binary<OP>::fwd(va.y, vb.y);
      r.z = Binary<OP>::fwd(va.z, vb.z);
      r.w = Binary<OP>::fwd(va.w, vb.w);
      reinterpret_cast<float4*>(out)[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = Binary<OP>::fwd(la(i), lb(i));
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = Binary<OP>::fwd(la(i), lb(i));
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) binary_fwd_general(const float* __restrict__ a, const float* __restrict__ b,
                                                                float* __restrict__ out, BcastGeom geo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < geo.numel; i += stride) {
    int64_t r = i, ia = 0, ib = 0;
#pragma unroll
    for (int d = RT_MAX_DIMS - 1; d >= 0; --d) {
      if (d < geo.nd) {
        int64_t c = r % geo.shape[d];
        r /= geo.shape[d];
        ia += c * geo.sa[d];
        ib += c * geo.sb[d];
      }
    }
    out[i] = Binary<OP>::fwd(a[ia], b[ib]);
  }
}

// Full-size products g*df (no reduction) for arbitrary broadcast geometry; used as
// the first step of the general backward path.  which: 0 -> da term, 1 -> db term.
template <int OP>
__global__ void __launch_bounds__(kThreads) binary_bwd_general_term(const float* __restrict__ a, const float* __restrict__ b,
                                                                     const float* __restrict__ g, float* __restrict__ out,
                                                                     BcastGeom geo, int which) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < geo.numel; i += stride) {
    int64_t r = i, ia = 0, ib = 0;
#pragma unroll
    for (int d = RT_MAX_DIMS - 1; d >= 0; --d) {
      if (d < geo.nd) {
        int64_t c = r % geo.shape[d];
        r /= geo.shape[d];
        ia += c * geo.sa[d];
        ib += c * geo.sb[d];
      }
    }
    float av = a[ia], bv = b[ib], gv = g[i];
    out[i] = which == 0 ? Binary<OP>::da(av, bv, gv) : Binary<OP>::db(av, bv, gv);
  }
}

// Same-shape backward: one pass reads g, a, b and writes da and/or db.
template <int OP, bool VEC>
__global__ void __launch_bounds__(kThreads) binary_bwd_same(const float* __restrict__ a, const float* __restrict__ b,
                                                             const float* __restrict__ g, float* __restrict__ da,
                                                             float* __restrict__ db, int64_t n) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 va = __ldg(reinterpret_cast<const float4*>(a) + i);
      float4 vb = __ldg(reinterpret_cast<const float4*>(b) + i);
      float4 vg = __ldg(reinterpret_cast<const float4*>(g) + i);
      if (da) {
        float4 r;
        r.x = Binary<OP>::da(va.x, vb.x, vg.x);
        r.y = Binary<OP>::da(va.y, vb.y, vg.y);
        r.z = Binary<OP>::da(va.z, vb.z, vg.z);
        r.w = Binary<OP>::da(va.w, vb.w, vg.w);
        reinterpret_cast<float4*>(da)[i] = r;
      }
      if (db) {
        float4 r;
        r.x = Binary<OP>::db(va.x, vb.x, vg.x);
        r.y = Binary<OP>::db(va.y, vb.y, vg.y);
        r.z = Binary<OP>::db(va.z, vb.z, vg.z);
        r.w = Binary<OP>::db(va.w, vb.w, vg.w);
        reinterpret_cast<float4*>(db)[i] = r;
      }
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
      if (da) da[i] = Binary<OP>::da(a[i], b[i], g[i]);
      if (db) db[i] = Binary<OP>::db(a[i], b[i], g[i]);
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      if (da) da[i] = Binary<OP>::da(a[i], b[i], g[i]);
      if (db) db[i] = Binary<OP>::db(a[i], b[i], g[i]);
    }
  }
}

// Row-vector broadcast backward: `full` is [rows, cols], `vec` is [cols] (or a
// scalar when cols == 1 is handled by the caller through the scalar kernel).
// One pass: d_full[r,c] is written, and the column sums of the vector-side term are
// reduced over the rows this block owns into partial[blockIdx.y, c].
// SWAP = false: a is the full operand, b the vector.  SWAP = true: the reverse.
constexpr int kColTile = 128;  // columns per block (32 threads x float4)
constexpr int kRowLanes = 8;   // threadIdx.y
template <int OP, bool SWAP>
__global__ void __launch_bounds__(kColTile / 4 * kRowLanes) binary_bwd_rowvec(
    const float* __restrict__ full, const float* __restrict__ vec, const float* __restrict__ g,
    float* __restrict__ d_full, float* __restrict__ partial, int64_t rows, int64_t cols, int rows_per_block) {
  __shared__ float4 red[kRowLanes][kColTile / 4];
  int c4 = blockIdx.x * (kColTile / 4) + threadIdx.x;  // float4 column index
  int64_t cols4 = cols >> 2;
  int64_t r0 = (int64_t)blockIdx.y * rows_per_block;
  int64_t r1 = r0 + rows_per_block;
  if (r1 > rows) r1 = rows;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c4 < cols4) {
    float4 v = __ldg(reinterpret_cast<const float4*>(vec) + c4);
    auto process = [&](int64_t idx, const float4& f, const float4& gg) {
      float4 df, dv;
      if (!SWAP) {
        df.x = Binary<OP>::da(f.x, v.x, gg.x); df.y = Binary<OP>::da(f.y, v.y, gg.y);
        df.z = Binary<OP>::da(f.z, v.z, gg.z); df.w = Binary<OP>::da(f.w, v.w, gg.w);
        dv.x = Binary<OP>::db(f.x, v.x, gg.x); dv.y = Binary<OP>::db(f.y, v.y, gg.y);
        dv.z = Binary<OP>::db(f.z, v.z, gg.z); dv.w = Binary<OP>::db(f.w, v.w, gg.w);
      } else {
        df.x = Binary<OP>::db(v.x, f.x, gg.x); df.y = Binary<OP>::db(v.y, f.y, gg.y);
        df.z = Binary<OP>::db(v.z, f.z, gg.z); df.w = Binary<OP>::db(v.w, f.w, gg.w);
        dv.x = Binary<OP>::da(v.x, f.x, gg.x); dv.y = Binary<OP>::da(v.y, f.y, gg.y);
        dv.z = Binary<OP>::da(v.z, f.z, gg.z); dv.w = Binary<OP>::da(v.w, f.w, gg.w);
      }
      if (d_full) reinterpret_cast<float4*>(d_full)[idx] = df;
      acc.x += dv.x; acc.y += dv.y; acc.z += dv.z; acc.w += dv.w;
    };
    int64_t r = r0 + threadIdx.y;
    // four rows per trip: eight independent 128-bit loads in flight per thread
    for (; r + 3 * kRowLanes < r1; r += 4 * kRowLanes) {
      float4 f[4], gg[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t idx = (r + u * kRowLanes) * cols4 + c4;
        f[u] = __ldg(reinterpret_cast<const float4*>(full) + idx);
        gg[u] = __ldg(reinterpret_cast<const float4*>(g) + idx);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) process((r + u * kRowLanes) * cols4 + c4, f[u], gg[u]);
    }
    for (; r < r1; r += kRowLanes) {
      const int64_t idx = r * cols4 + c4;
      process(idx, __ldg(reinterpret_cast<const float4*>(full) + idx), __ldg(reinterpret_cast<const float4*>(g) + idx));
    }
  }
  if (partial == nullptr) return;
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c4 < cols4) {
    float4 s = red[0][threadIdx.x];
#pragma unroll
    for (int j = 1; j < kRowLanes; ++j) {
      float4 t = red[j][threadIdx.x];
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    reinterpret_cast<float4*>(partial)[(int64_t)blockIdx.y * cols4 + c4] = s;
  }
}

// Scalar broadcast backward: `full` [n] against a one-element operand.  Writes
// d_full and one partial sum per block of the scalar-side term.
template <int OP, bool SWAP>
__global__ void __launch_bounds__(kThreads) binary_bwd_scalar(const float* __restrict__ full, const float* __restrict__ sc,
                                                               const float* __restrict__ g, float* __restrict__ d_full,
                                                               float* __restrict__ partial, int64_t n) {
  __shared__ float red[kThreads / 32];
  float s = sc[0];
  float acc = 0.f;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float f = full[i], gg = g[i];
    float df = SWAP ? Binary<OP>::db(s, f, gg) : Binary<OP>::da(f, s, gg);
    float ds = SWAP ? Binary<OP>::da(s, f, gg) : Binary<OP>::db(f, s, gg);
    if (d_full) d_full[i] = df;
    acc += ds;
  }
  if (partial == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) partial[blockIdx.x] = v;
  }
}

__global__ void __launch_bounds__(kThreads) fill_kernel(float* __restrict__ dst, float v, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (rt_aligned16(dst)) {
    int64_t n4 = n >> 2;
    float4 v4 = make_float4(v, v, v, v);
    for (int64_t i = tid; i < n4; i += stride) reinterpret_cast<float4*>(dst)[i] = v4;
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) dst[i] = v;
  } else {
    for (int64_t i = tid; i < n; i += stride) dst[i] = v;
  }
}

__global__ void __launch_bounds__(kThreads) broadcast_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                              BcastGeom geo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < geo.numel; i += stride) {
    int64_t r = i, ia = 0;
#pragma unroll
    for (int d = RT_MAX_DIMS - 1; d >= 0; --d) {
      if (d < geo.nd) {
        int64_t c = r % geo.shape[d];
        r /= geo.shape[d];
        ia += c * geo.sa[d];
      }
    }
    out[i] = x[ia];
  }
}

// 32x32 shared-memory tile transpose (padded against bank conflicts).
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                         int64_t rows, int64_t cols) {
  __shared__ float tile[32][33];
  int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = x[r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[c * rows + r] = tile[threadIdx.x][j];
  }
}

// Copies a box between a small tensor (box-shaped, contiguous) and a window of a
// larger one.  TO_BIG: big[starts + i] = small[i]; else small[i] = big[starts + i].
struct BoxGeom {
  int nd;
  int64_t box[RT_MAX_DIMS];        // box extents (outermost first)
  int64_t big_stride[RT_MAX_DIMS]; // element strides of the big tensor
  int64_t big_offset;              // offset of the window origin
  int64_t numel;
};
template <bool TO_BIG>
__global__ void __launch_bounds__(kThreads) box_copy_kernel(float* __restrict__ big, float* __restrict__ small_, BoxGeom geo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < geo.numel; i += stride) {
    int64_t r = i, off = geo.big_offset;
#pragma unroll
    for (int d = RT_MAX_DIMS - 1; d >= 0; --d) {
      if (d < geo.nd) {
        int64_t c = r % geo.box[d];
        r /= geo.box[d];
        off += c * geo.big_stride[d];
      }
    }
    if (TO_BIG) big[off] = small_[i];
    else small_[i] = big[off];
  }
}

// Builds the collapsed broadcast geometry of two right-aligned shapes.
// Returns false when the shapes are not broadcast-compatible.
bool make_geom(const int64_t* as, int and_, const int64_t* bs, int bnd, BcastGeom* geo, int64_t* out_shape, int* out_nd) {
  int nd = and_ > bnd ? and_ : bnd;
  if (nd > RT_MAX_DIMS) return false;
  int64_t A[RT_MAX_DIMS], Bv[RT_MAX_DIMS], O[RT_MAX_DIMS];
  for (int i = 0; i < nd; ++i) {
    A[i] = i < nd - and_ ? 1 : as[i - (nd - and_)];
    Bv[i] = i < nd - bnd ? 1 : bs[i - (nd - bnd)];
    if (A[i] == Bv[i]) O[i] = A[i];
    else if (A[i] == 1) O[i] = Bv[i];
    else if (Bv[i] == 1) O[i] = A[i];
    else return false;
  }
  if (out_shape) {
    for (int i = 0; i < nd; ++i) out_shape[i] = O[i];
    *out_nd = nd;
  }
  int64_t sa[RT_MAX_DIMS], sb[RT_MAX_DIMS];
  int64_t ra = 1, rb = 1;
  for (int i = nd - 1; i >= 0; --i) {
    sa[i] = (A[i] == 1 && O[i] != 1) ? 0 : ra;
    sb[i] = (Bv[i] == 1 && O[i] != 1) ? 0 : rb;
    ra *= A[i];
    rb *= Bv[i];
  }
  // collapse: drop size-1 dims, merge neighbours that are contiguous for both operands
  geo->nd = 0;
  geo->numel = 1;
  for (int i = 0; i < nd; ++i) {
    geo->numel *= O[i];
    if (O[i] == 1) continue;
    if (geo->nd > 0) {
      int p = geo->nd - 1;
      if (geo->sa[p] == sa[i] * O[i] && geo->sb[p] == sb[i] * O[i]) {
        geo->shape[p] *= O[i];
        geo->sa[p] = sa[i];
        geo->sb[p] = sb[i];
        continue;
      }
    }
    geo->shape[geo->nd] = O[i];
    geo->sa[geo->nd] = sa[i];
    geo->sb[geo->nd] = sb[i];
    geo->nd++;
  }
  return true;
}

int64_t numel_of(const int64_t* s, int nd) {
  int64_t n = 1;
  for (int i = 0; i < nd; ++i) n *= s[i];
  return n;
}

// Classification of the collapsed geometry.
enum BMode { BM_SAME = 0, BM_B_SCALAR = 1, BM_A_SCALAR = 2, BM_B_ROWVEC = 3, BM_A_ROWVEC = 4, BM_GENERAL = 5 };
BMode classify(const BcastGeom& g, int64_t* cols) {
  *cols = 1;
  if (g.nd == 0) return BM_SAME;
  if (g.nd == 1) {
    if (g.sa[0] == 1 && g.sb[0] == 1) return BM_SAME;
    if (g.sa[0] == 1 && g.sb[0] == 0) return BM_B_SCALAR;
    if (g.sa[0] == 0 && g.sb[0] == 1) return BM_A_SCALAR;
  }
  if (g.nd == 2) {
    *cols = g.shape[1];
    if (g.sa[0] == g.shape[1] && g.sa[1] == 1 && g.sb[0] == 0 && g.sb[1] == 1) return BM_B_ROWVEC;
    if (g.sb[0] == g.shape[1] && g.sb[1] == 1 && g.sa[0] == 0 && g.sa[1] == 1) return BM_A_ROWVEC;
  }
  return BM_GENERAL;
}

template <int OP>
rt_status binary_forward(rt_ctx* ctx, const float* a, const float* b, float* out, const BcastGeom& geo) {
  int64_t cols;
  BMode m = classify(geo, &cols);
  int64_t n = geo.numel;
  bool al = rt_aligned16(a) && rt_aligned16(b) && rt_aligned16(out);
  int gridv = rt_grid_for(ctx, (n + 3) / 4, kThreads * 2), grids = rt_grid_for(ctx, n, kThreads * 2);
#define RT_FAST(MODE, VECOK)                                                                            \
  if (al && (VECOK)) binary_fwd_fast<OP, MODE, true><<<gridv, kThreads, 0, ctx->stream>>>(a, b, out, n, cols); \
  else binary_fwd_fast<OP, MODE, false><<<grids, kThreads, 0, ctx->stream>>>(a, b, out, n, cols);
  switch (m) {
    case BM_SAME: RT_FAST(0, true) break;
    case BM_B_SCALAR: RT_FAST(1, true) break;
    case BM_A_SCALAR: RT_FAST(2, true) break;
    case BM_B_ROWVEC: RT_FAST(3, cols % 4 == 0) break;
    case BM_A_ROWVEC: RT_FAST(4, cols % 4 == 0) break;
    default: binary_fwd_general<OP><<<grids, kThreads, 0, ctx->stream>>>(a, b, out, geo);
  }
#undef RT_FAST
  RT_LAUNCHED(ctx);
  return RT_OK;
}

}  // namespace

// Declared in k_reduce.cu: out[o,i] = sum_k x[o,k,i] (deterministic two-pass when split).
rt_status rt_sum_axis_internal(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out,
                               float scale);

namespace {

template <int OP>
rt_status binary_backward(rt_ctx* ctx, const float* a, const int64_t* as, int and_, const float* b, const int64_t* bs,
                          int bnd, const float* g, float* da, float* db, const BcastGeom& geo, const int64_t* out_shape,
                          int out_nd) {
  int64_t cols;
  BMode m = classify(geo, &cols);
  int64_t n = geo.numel;
  if (m == BM_SAME) {
    bool al = rt_aligned16(a) && rt_aligned16(b) && rt_aligned16(g) && (!da || rt_aligned16(da)) && (!db || rt_aligned16(db));
    if (al) binary_bwd_same<OP, true><<<rt_grid_for(ctx, (n + 3) / 4, kThreads * 2), kThreads, 0, ctx->stream>>>(a, b, g, da, db, n);
    else binary_bwd_same<OP, false><<<rt_grid_for(ctx, n, kThreads * 2), kThreads, 0, ctx->stream>>>(a, b, g, da, db, n);
    RT_LAUNCHED(ctx);
    return RT_OK;
  }
  if (m == BM_B_SCALAR || m == BM_A_SCALAR) {
    const bool swap = (m == BM_A_SCALAR);
    const float* full = swap ? b : a;
    const float* sc = swap ? a : b;
    float* d_full = swap ? db : da;
    float* d_sc = swap ? da : db;
    int grid = rt_grid_for(ctx, n, kThreads * 4, 4);
    RtScratch part(ctx);
    if (d_sc) {
      rt_status st = part.alloc(sizeof(float) * grid);
      if (st != RT_OK) return st;
    }
    if (swap) binary_bwd_scalar<OP, true><<<grid, kThreads, 0, ctx->stream>>>(full, sc, g, d_full, part.as<float>(), n);
    else binary_bwd_scalar<OP, false><<<grid, kThreads, 0, ctx->stream>>>(full, sc, g, d_full, part.as<float>(), n);
    RT_LAUNCHED(ctx);
    if (d_sc) return rt_sum_axis_internal(ctx, part.as<float>(), 1, grid, 1, d_sc, 1.f);
    return RT_OK;
  }
  if ((m == BM_B_ROWVEC || m == BM_A_ROWVEC) && cols % 4 == 0) {
    const bool swap = (m == BM_A_ROWVEC);
    const float* full = swap ? b : a;
    const float* vec = swap ? a : b;
    float* d_full = swap ? db : da;
    float* d_vec = swap ? da : db;
    if (rt_aligned16(full) && rt_aligned16(vec) && rt_aligned16(g) && (!d_full || rt_aligned16(d_full))) {
      int64_t rows = geo.shape[0];
      int col_blocks = (int)((cols + kColTile - 1) / kColTile);
      // enough row chunks to fill the machine, at least kRowLanes*4 rows each
      int64_t want = ((int64_t)ctx->sm_count * 4 + col_blocks - 1) / col_blocks;
      int64_t max_chunks = (rows + kRowLanes * 4 - 1) / (kRowLanes * 4);
      int64_t chunks = want < max_chunks ? want : max_chunks;
      if (chunks < 1) chunks = 1;
      if (chunks > 65535) chunks = 65535;
      int rpb = (int)((rows + chunks - 1) / chunks);
      chunks = (rows + rpb - 1) / rpb;
      RtScratch part(ctx);
      if (d_vec) {
        rt_status st = part.alloc(sizeof(float) * chunks * cols);
        if (st != RT_OK) return st;
      }
      dim3 grid(col_blocks, (unsigned)chunks), block(kColTile / 4, kRowLanes);
      if (swap) binary_bwd_rowvec<OP, true><<<grid, block, 0, ctx->stream>>>(full, vec, g, d_full, part.as<float>(), rows, cols, rpb);
      else binary_bwd_rowvec<OP, false><<<grid, block, 0, ctx->stream>>>(full, vec, g, d_full, part.as<float>(), rows, cols, rpb);
      RT_LAUNCHED(ctx);
      if (d_vec) return rt_sum_axis_internal(ctx, part.as<float>(), 1, chunks, cols, d_vec, 1.f);
      return RT_OK;
    }
  }
  // General path: full-size term, then un-broadcast down to the operand's shape.
  int grid = rt_grid_for(ctx, n, kThreads * 2);
  for (int which = 0; which < 2; ++which) {
    float* dst = which == 0 ? da : db;
    if (!dst) continue;
    const int64_t* ts = which == 0 ? as : bs;
    int tnd = which == 0 ? and_ : bnd;
    bool full_shape = numel_of(ts, tnd) == n;
    RtScratch tmp(ctx);
    float* term = dst;
    if (!full_shape) {
      rt_status st = tmp.alloc(sizeof(float) * n);
      if (st != RT_OK) return st;
      term = tmp.as<float>();
    }
    binary_bwd_general_term<OP><<<grid, kThreads, 0, ctx->stream>>>(a, b, g, term, geo, which);
    RT_LAUNCHED(ctx);
    if (!full_shape) {
      rt_status st = rt_unbroadcast(ctx, term, out_shape, out_nd, ts, tnd, dst);
      if (st != RT_OK) return st;
    }
  }
  return RT_OK;
}

}  // namespace

// Row gather: one thread per 16 bytes (or per element when rows are not 16-byte multiples) of the output.
template <bool VEC>
__global__ void __launch_bounds__(kThreads) gather_rows_kernel(const float* __restrict__ src, int64_t rows, int64_t row_len,
                                                               const int32_t* __restrict__ idx, int64_t n_idx, float* __restrict__ out) {
  const int64_t per_row = VEC ? row_len / 4 : row_len;
  const int64_t total = n_idx * per_row;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / per_row, c = t - i * per_row;
    const int64_t r = __ldg(idx + i);
    const bool ok = r >= 0 && r < rows;
    if (VEC) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) v = __ldg(reinterpret_cast<const float4*>(src + r * row_len) + c);
      reinterpret_cast<float4*>(out + i * row_len)[c] = v;
    } else {
      out[i * row_len + c] = ok ? __ldg(src + r * row_len + c) : 0.f;
    }
  }
}

extern "C" {

rt_status rt_fill(rt_ctx* ctx, float* dst, float value, int64_t n) {
  RT_CHECK_CTX(ctx);
  if (n <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, dst);
  if (value == 0.f) {
    RT_CUDA(ctx, cudaMemsetAsync(dst, 0, sizeof(float) * n, ctx->stream));
    return RT_OK;
  }
  fill_kernel<<<rt_grid_for(ctx, (n + 3) / 4, kThreads * 2), kThreads, 0, ctx->stream>>>(dst, value, n);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_unary(rt_ctx* ctx, int op, const float* x, float* y, int64_t n, float p0, float p1) {
  RT_CHECK_CTX(ctx);
  if (op < 0 || op >= RT_UNARY_COUNT) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_unary: unknown op %d", op);
  if (op == RT_DIV_SCALAR && p0 == 0.f) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "Division by zero scalar");
  if (op == RT_CLIP && p0 > p1) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "Clip min_val cannot be greater than max_val");
  if (n <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, y);
  switch (op) {
#define RT_CASE(OPC) case OPC: launch_unary_fwd<OPC>(ctx, x, y, n, p0, p1); break;
    RT_CASE(RT_RELU) RT_CASE(RT_ELU) RT_CASE(RT_EXP) RT_CASE(RT_LN) RT_CASE(RT_SIN) RT_CASE(RT_TANH)
    RT_CASE(RT_SIGMOID) RT_CASE(RT_SOFTPLUS) RT_CASE(RT_SQUARE) RT_CASE(RT_SQRT) RT_CASE(RT_ABS) RT_CASE(RT_CLIP)
    RT_CASE(RT_MUL_SCALAR) RT_CASE(RT_DIV_SCALAR) RT_CASE(RT_COS) RT_CASE(RT_TAN)
#undef RT_CASE
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_unary_backward(rt_ctx* ctx, int op, const float* x, const float* g, float* dx, int64_t n, float p0, float p1) {
  RT_CHECK_CTX(ctx);
  if (op < 0 || op >= RT_UNARY_COUNT) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_unary_backward: unknown op %d", op);
  if (op == RT_DIV_SCALAR && p0 == 0.f) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "Division by zero scalar");
  if (n <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, g);
  RT_CHECK_PTR(ctx, dx);
  switch (op) {
#define RT_CASE(OPC) case OPC: launch_unary_bwd<OPC>(ctx, x, g, dx, n, p0, p1); break;
    RT_CASE(RT_RELU) RT_CASE(RT_ELU) RT_CASE(RT_EXP) RT_CASE(RT_LN) RT_CASE(RT_SIN) RT_CASE(RT_TANH)
    RT_CASE(RT_SIGMOID) RT_CASE(RT_SOFTPLUS) RT_CASE(RT_SQUARE) RT_CASE(RT_SQRT) RT_CASE(RT_ABS) RT_CASE(RT_CLIP)
    RT_CASE(RT_MUL_SCALAR) RT_CASE(RT_DIV_SCALAR) RT_CASE(RT_COS) RT_CASE(RT_TAN)
#undef RT_CASE
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_binary(rt_ctx* ctx, int op, const float* a, const int64_t* a_shape, int a_ndim, const float* b,
                    const int64_t* b_shape, int b_ndim, float* out) {
  RT_CHECK_CTX(ctx);
  if (op < 0 || op >= RT_BINARY_COUNT) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_binary: unknown op %d", op);
  if (a_ndim < 0 || b_ndim < 0 || a_ndim > RT_MAX_DIMS || b_ndim > RT_MAX_DIMS)
    RT_FAIL(ctx, RT_ERR_DIMENSION_MISMATCH, "rt_binary: at most %d dimensions", RT_MAX_DIMS);
  BcastGeom geo;
  if (!make_geom(a_shape, a_ndim, b_shape, b_ndim, &geo, nullptr, nullptr))
    RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_binary: shapes cannot be broadcast together");
  if (geo.numel == 0) return RT_OK;
  RT_CHECK_PTR(ctx, a);
  RT_CHECK_PTR(ctx, b);
  RT_CHECK_PTR(ctx, out);
  switch (op) {
#define RT_CASE(OPC) case OPC: return binary_forward<OPC>(ctx, a, b, out, geo);
    RT_CASE(RT_ADD) RT_CASE(RT_SUB) RT_CASE(RT_MUL) RT_CASE(RT_DIV) RT_CASE(RT_POWF) RT_CASE(RT_MAXIMUM)
    RT_CASE(RT_MINIMUM) RT_CASE(RT_EQUAL) RT_CASE(RT_NOT_EQUAL) RT_CASE(RT_GREATER) RT_CASE(RT_GREATER_EQUAL)
    RT_CASE(RT_LESS) RT_CASE(RT_LESS_EQUAL)
#undef RT_CASE
  }
  return RT_ERR_INTERNAL;
}

rt_status rt_binary_backward(rt_ctx* ctx, int op, const float* a, const int64_t* a_shape, int a_ndim, const float* b,
                             const int64_t* b_shape, int b_ndim, const float* g, float* da, float* db) {
  RT_CHECK_CTX(ctx);
  if (op < 0 || op > RT_MINIMUM) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_binary_backward: op %d has no gradient", op);
  if (a_ndim < 0 || b_ndim < 0 || a_ndim > RT_MAX_DIMS || b_ndim > RT_MAX_DIMS)
    RT_FAIL(ctx, RT_ERR_DIMENSION_MISMATCH, "rt_binary_backward: at most %d dimensions", RT_MAX_DIMS);
  BcastGeom geo;
  int64_t out_shape[RT_MAX_DIMS];
  int out_nd = 0;
  if (!make_geom(a_shape, a_ndim, b_shape, b_ndim, &geo, out_shape, &out_nd))
    RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_binary_backward: shapes cannot be broadcast together");
  if (!da && !db) return RT_OK;
  if (geo.numel == 0) {  // an empty broadcast result still owes zero gradients to non-empty operands
    rt_status st = da ? rt_fill(ctx, da, 0.f, numel_of(a_shape, a_ndim)) : RT_OK;
    if (st == RT_OK && db) st = rt_fill(ctx, db, 0.f, numel_of(b_shape, b_ndim));
    return st;
  }
  RT_CHECK_PTR(ctx, a);
  RT_CHECK_PTR(ctx, b);
  RT_CHECK_PTR(ctx, g);
  switch (op) {
#define RT_CASE(OPC) \
  case OPC: return binary_backward<OPC>(ctx, a, a_shape, a_ndim, b, b_shape, b_ndim, g, da, db, geo, out_shape, out_nd);
    RT_CASE(RT_ADD) RT_CASE(RT_SUB) RT_CASE(RT_MUL) RT_CASE(RT_DIV) RT_CASE(RT_POWF) RT_CASE(RT_MAXIMUM) RT_CASE(RT_MINIMUM)
#undef RT_CASE
  }
  return RT_ERR_INTERNAL;
}

rt_status rt_unbroadcast(rt_ctx* ctx, const float* g, const int64_t* g_shape, int g_ndim, const int64_t* t_shape,
                         int t_ndim, float* out) {
  RT_CHECK_CTX(ctx);
  if (g_ndim > RT_MAX_DIMS || t_ndim > g_ndim)
    RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_unbroadcast: target has more dimensions than the gradient");
  // right-align the target; mark reduced dims
  int64_t cur[RT_MAX_DIMS];
  bool red[RT_MAX_DIMS];
  int nd = g_ndim;
  int64_t n = 1;
  bool any = false;
  for (int i = 0; i < nd; ++i) {
    cur[i] = g_shape[i];
    n *= cur[i];
    int ti = i - (nd - t_ndim);
    int64_t td = ti < 0 ? 1 : t_shape[ti];
    if (ti < 0) red[i] = true;
    else if (td == cur[i]) red[i] = false;
    else if (td == 1) red[i] = true;
    else RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_unbroadcast: dimension %d: %lld cannot reduce to %lld", i, (long long)cur[i], (long long)td);
    if (red[i] && cur[i] != 1) any = true;
  }
  if (n == 0) return out ? rt_fill(ctx, out, 0.f, numel_of(t_shape, t_ndim)) : RT_OK;
  RT_CHECK_PTR(ctx, g);
  RT_CHECK_PTR(ctx, out);
  if (!any) return rt_memcpy_d2d(ctx, out, g, sizeof(float) * n);
  // Reduce one contiguous group of reduced dims at a time, innermost group first.
  const float* src = g;
  RtScratch tmpA(ctx), tmpB(ctx);
  int end = nd;
  bool use_a = true;
  while (true) {
    // find the last group of reduced dims (with extent > 1) before `end`
    int hi = end - 1;
    while (hi >= 0 && !(red[hi] && cur[hi] != 1)) --hi;
    if (hi < 0) break;
    int lo = hi;
    while (lo - 1 >= 0 && (red[lo - 1] || cur[lo - 1] == 1)) --lo;
    int64_t outer = 1, len = 1, inner = 1;
    for (int i = 0; i < lo; ++i) outer *= cur[i];
    for (int i = lo; i <= hi; ++i) len *= cur[i];
    for (int i = hi + 1; i < nd; ++i) inner *= cur[i];
    // is this the last group?
    bool more = false;
    for (int i = 0; i < lo; ++i)
      if (red[i] && cur[i] != 1) more = true;
    float* dst = out;
    if (more) {
      RtScratch& t = use_a ? tmpA : tmpB;
      if (t.ptr) { rt_free(ctx, t.ptr); t.ptr = nullptr; }
      rt_status st = t.alloc(sizeof(float) * outer * inner);
      if (st != RT_OK) return st;
      dst = t.as<float>();
      use_a = !use_a;
    }
    rt_status st = rt_sum_axis_internal(ctx, src, outer, len, inner, dst, 1.f);
    if (st != RT_OK) return st;
    for (int i = lo; i <= hi; ++i) cur[i] = 1;
    src = dst;
    end = lo;
    if (!more) break;
  }
  return RT_OK;
}

rt_status rt_broadcast_to(rt_ctx* ctx, const float* x, const int64_t* x_shape, int x_ndim, const int64_t* out_shape,
                          int out_ndim, float* out) {
  RT_CHECK_CTX(ctx);
  if (out_ndim > RT_MAX_DIMS || x_ndim > out_ndim)
    RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_broadcast_to: cannot broadcast to fewer dimensions");
  for (int i = 0; i < x_ndim; ++i) {
    int64_t od = out_shape[i + (out_ndim - x_ndim)];
    if (x_shape[i] != od && x_shape[i] != 1)
      RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_broadcast_to: dimension %d: %lld -> %lld", i, (long long)x_shape[i], (long long)od);
  }
  BcastGeom geo;
  if (!make_geom(x_shape, x_ndim, out_shape, out_ndim, &geo, nullptr, nullptr))
    RT_FAIL(ctx, RT_ERR_INCOMPATIBLE_SHAPES, "rt_broadcast_to: incompatible shapes");
  if (geo.numel == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, out);
  if (numel_of(x_shape, x_ndim) == geo.numel) return rt_memcpy_d2d(ctx, out, x, sizeof(float) * geo.numel);
  broadcast_kernel<<<rt_grid_for(ctx, geo.numel, kThreads * 2), kThreads, 0, ctx->stream>>>(x, out, geo);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_transpose2d(rt_ctx* ctx, const float* x, int64_t rows, int64_t cols, float* out) {
  RT_CHECK_CTX(ctx);
  if (rows <= 0 || cols <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, out);
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32)), block(32, 8);
  if (grid.y > 65535) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_transpose2d: too many rows");
  transpose_kernel<<<grid, block, 0, ctx->stream>>>(x, out, rows, cols);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

static rt_status make_box(rt_ctx* ctx, const int64_t* big_shape, int ndim, const int64_t* starts, const int64_t* box_shape,
                          BoxGeom* geo) {
  if (ndim < 0 || ndim > RT_MAX_DIMS) RT_FAIL(ctx, RT_ERR_DIMENSION_MISMATCH, "slice: at most %d dimensions", RT_MAX_DIMS);
  geo->nd = ndim;
  geo->numel = 1;
  geo->big_offset = 0;
  int64_t s = 1;
  for (int i = ndim - 1; i >= 0; --i) {
    if (starts[i] < 0 || box_shape[i] < 0 || starts[i] + box_shape[i] > big_shape[i])
      RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "slice: range out of bounds in dimension %d", i);
    geo->box[i] = box_shape[i];
    geo->big_stride[i] = s;
    geo->big_offset += starts[i] * s;
    geo->numel *= box_shape[i];
    s *= big_shape[i];
  }
  return RT_OK;
}

rt_status rt_slice_assign(rt_ctx* ctx, float* dst, const int64_t* dst_shape, int ndim, const int64_t* starts,
                          const float* src, const int64_t* src_shape) {
  RT_CHECK_CTX(ctx);
  BoxGeom geo;
  rt_status st = make_box(ctx, dst_shape, ndim, starts, src_shape, &geo);
  if (st != RT_OK) return st;
  if (geo.numel == 0) return RT_OK;
  RT_CHECK_PTR(ctx, dst);
  RT_CHECK_PTR(ctx, src);
  box_copy_kernel<true><<<rt_grid_for(ctx, geo.numel, kThreads * 2), kThreads, 0, ctx->stream>>>(dst, const_cast<float*>(src), geo);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_slice(rt_ctx* ctx, const float* x, const int64_t* x_shape, int ndim, const int64_t* starts,
                   const int64_t* out_shape, float* out) {
  RT_CHECK_CTX(ctx);
  BoxGeom geo;
  rt_status st = make_box(ctx, x_shape, ndim, starts, out_shape, &geo);
  if (st != RT_OK) return st;
  if (geo.numel == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, out);
  box_copy_kernel<false><<<rt_grid_for(ctx, geo.numel, kThreads * 2), kThreads, 0, ctx->stream>>>(const_cast<float*>(x), out, geo);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// out[i, :] = src[idx[i], :] for i < n_idx: the batch gather of data::get_random_batch (src/data.rs:125-209), which in the
// reference copies the whole data set to the host, picks the rows there and uploads the batch.  `idx` is a device array;
// an index outside [0, rows) (the host wrapper has already refused it) yields a row of zeros.
rt_status rt_gather_rows(rt_ctx* ctx, const float* src, int64_t rows, int64_t row_len, const int32_t* idx, int64_t n_idx, float* out) {
  RT_CHECK_CTX(ctx);
  if (rows < 0 || row_len < 0 || n_idx < 0) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_gather_rows: negative size");
  if (n_idx == 0 || row_len == 0) return RT_OK;
  RT_CHECK_PTR(ctx, src);
  RT_CHECK_PTR(ctx, idx);
  RT_CHECK_PTR(ctx, out);
  if (rows >= (1ll << 31) || n_idx * row_len >= (1ll << 40)) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_gather_rows: size out of range");
  const bool vec = (row_len % 4 == 0) && rt_aligned16(src) && rt_aligned16(out);
  const int64_t work = n_idx * (vec ? row_len / 4 : row_len);
  if (vec)
    gather_rows_kernel<true><<<rt_grid_for(ctx, work, kThreads), kThreads, 0, ctx->stream>>>(src, rows, row_len, idx, n_idx, out);
  else
    gather_rows_kernel<false><<<rt_grid_for(ctx, work, kThreads), kThreads, 0, ctx->stream>>>(src, rows, row_len, idx, n_idx, out);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

}  // extern "C"
