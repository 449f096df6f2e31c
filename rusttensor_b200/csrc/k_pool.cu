// max_pool2d forward (values + in-window argmax index stored as f32) and backward
// (gradient routed through the saved indices).
//
// Index semantics follow the reference CPU code bit for bit (src/ops/cpu_ops.rs:7-61):
// windows are scanned ky-outer / kx-inner, a candidate wins only with a strict `>`, the
// running maximum starts at -inf with index 0, out-of-range taps read as -inf (so they
// can never win), NaN never wins.
//
// Backward (src/ops/cpu_backward.rs:9-46): when windows do not overlap (stride >= kernel)
// every input element belongs to at most one window, so the scatter has no write
// conflicts and runs without atomics; the common 2x2 / stride 2 / no-padding case is
// written as a gather that produces each 2x2 block of dx with two 8-byte stores and needs
// no zero-fill.  Overlapping windows are gathered per input element in the reference's order of additions.
#include <cmath>

#include "rt_internal.cuh"

namespace {

constexpr int kThreads = 256;

template <bool RELU>  // RELU: the pooled tensor is relu(x), computed on the fly (fused relu + max_pool2d)
__global__ void __launch_bounds__(kThreads) pool_fwd_general(const float* __restrict__ x, float* __restrict__ y,
                                                              float* __restrict__ idx, int64_t total, int h, int w, int ho,
                                                              int wo, int kh, int kw, int sh, int sw, int ph, int pw) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
    int xo = (int)(o % wo);
    int64_t r = o / wo;
    int yo = (int)(r % ho);
    int64_t bc = r / ho;
    const float* p = x + bc * h * w;
    float mv = -INFINITY;
    int mi = 0, iw = 0;
    for (int ky = 0; ky < kh; ++ky) {
      int iy = yo * sh + ky - ph;
      for (int kx = 0; kx < kw; ++kx, ++iw) {
        int ix = xo * sw + kx - pw;
        float v = -INFINITY;
        if (iy >= 0 && iy < h && ix >= 0 && ix < w) {
          v = __ldg(p + (int64_t)iy * w + ix);
          if (RELU) v = fmaxf(v, 0.f);
        }
        if (v > mv) {
          mv = v;
          mi = iw;
        }
      }
    }
    y[o] = mv;
    idx[o] = (float)mi;
  }
}

// 2x2 window, stride 2, no padding, even H and W: one thread per output, two 8-byte loads.
template <bool RELU>
__global__ void __launch_bounds__(kThreads) pool_fwd_2x2(const float* __restrict__ x, float* __restrict__ y,
                                                          float* __restrict__ idx, int64_t total, int w, int ho, int wo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
    int xo = (int)(o % wo);
    int64_t row = o / wo;  // = bc * ho + yo ; the input row pair starts at 2 * row (H = 2 * ho)
    const float2* p = reinterpret_cast<const float2*>(x + (row * 2) * w) + xo;
    float2 a = __ldg(p), b = __ldg(p + (w >> 1));
    if (RELU) {
      a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f);
      b.x = fmaxf(b.x, 0.f); b.y = fmaxf(b.y, 0.f);
    }
    float mv = -INFINITY;
    int mi = 0;
    if (a.x > mv) { mv = a.x; mi = 0; }
    if (a.y > mv) { mv = a.y; mi = 1; }
    if (b.x > mv) { mv = b.x; mi = 2; }
    if (b.y > mv) { mv = b.y; mi = 3; }
    y[o] = mv;
    idx[o] = (float)mi;
  }
}

template <bool RELU>  // RELU: dx is also masked with x > 0 (backward of the fused relu + max_pool2d)
__global__ void __launch_bounds__(kThreads) pool_bwd_2x2(const float* __restrict__ g, const float* __restrict__ idx,
                                                          const float* __restrict__ x, float* __restrict__ dx, int64_t total,
                                                          int w, int ho, int wo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
    int xo = (int)(o % wo);
    int64_t row = o / wo;
    float gv = __ldg(g + o);
    int mi = (int)lrintf(__ldg(idx + o));
    float2 a = make_float2(mi == 0 ? gv : 0.f, mi == 1 ? gv : 0.f);
    float2 b = make_float2(mi == 2 ? gv : 0.f, mi == 3 ? gv : 0.f);
    if (RELU) {
      const float2* q = reinterpret_cast<const float2*>(x + (row * 2) * w) + xo;
      const float2 xa = __ldg(q), xb = __ldg(q + (w >> 1));
      a.x = xa.x > 0.f ? a.x : 0.f; a.y = xa.y > 0.f ? a.y : 0.f;
      b.x = xb.x > 0.f ? b.x : 0.f; b.y = xb.y > 0.f ? b.y : 0.f;
    }
    float2* p = reinterpret_cast<float2*>(dx + (row * 2) * w) + xo;
    p[0] = a;
    p[w >> 1] = b;
  }
}

// The same with two neighbouring windows per thread: 64-bit loads of g and of the indices, 128-bit stores (wo even,
// 16-byte aligned rows).
template <bool RELU>
__global__ void __launch_bounds__(kThreads) pool_bwd_2x2_pair(const float* __restrict__ g, const float* __restrict__ idx,
                                                               const float* __restrict__ x, float* __restrict__ dx,
                                                               int64_t total2, int w, int wo2) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total2; o += stride) {
    const int xo = (int)(o % wo2);
    const int64_t row = o / wo2;
    const float2 gv = __ldcs(reinterpret_cast<const float2*>(g) + o);  // read once: streaming loads
    const float2 iv = __ldcs(reinterpret_cast<const float2*>(idx) + o);
    const int m0 = (int)lrintf(iv.x), m1 = (int)lrintf(iv.y);
    float4 a = make_float4(m0 == 0 ? gv.x : 0.f, m0 == 1 ? gv.x : 0.f, m1 == 0 ? gv.y : 0.f, m1 == 1 ? gv.y : 0.f);
    float4 b = make_float4(m0 == 2 ? gv.x : 0.f, m0 == 3 ? gv.x : 0.f, m1 == 2 ? gv.y : 0.f, m1 == 3 ? gv.y : 0.f);
    if (RELU) {
      const float4* q = reinterpret_cast<const float4*>(x + (row * 2) * w) + xo;
      const float4 xa = __ldg(q), xb = __ldg(q + (w >> 2));
      a.x = xa.x > 0.f ? a.x : 0.f; a.y = xa.y > 0.f ? a.y : 0.f; a.z = xa.z > 0.f ? a.z : 0.f; a.w = xa.w > 0.f ? a.w : 0.f;
      b.x = xb.x > 0.f ? b.x : 0.f; b.y = xb.y > 0.f ? b.y : 0.f; b.z = xb.z > 0.f ? b.z : 0.f; b.w = xb.w > 0.f ? b.w : 0.f;
    }
    float4* p = reinterpret_cast<float4*>(dx + (row * 2) * w) + xo;
    p[0] = a;
    p[w >> 2] = b;
  }
}

// Backward of max_pool2d(relu(.)) for 2x2 / stride 2 from the POOLED output: the gradient of window o goes to its saved
// position when y[o] > 0 (y = relu of the window's maximum, so y > 0 exactly when the input at that position was positive)
// and nowhere otherwise.  Two windows per thread like pool_bwd_2x2_pair; the un-pooled tensor is not read.
__global__ void __launch_bounds__(kThreads) pool_bwd_2x2_from_output(const float* __restrict__ y, const float* __restrict__ g,
                                                                      const float* __restrict__ idx, float* __restrict__ dx,
                                                                      int64_t total2, int w, int wo2) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total2; o += stride) {
    const int xo = (int)(o % wo2);
    const int64_t row = o / wo2;
    float2 gv = __ldcs(reinterpret_cast<const float2*>(g) + o);
    const float2 iv = __ldcs(reinterpret_cast<const float2*>(idx) + o);
    const float2 yv = __ldg(reinterpret_cast<const float2*>(y) + o);
    gv.x = yv.x > 0.f ? gv.x : 0.f;
    gv.y = yv.y > 0.f ? gv.y : 0.f;
    const int m0 = (int)lrintf(iv.x), m1 = (int)lrintf(iv.y);
    const float4 a = make_float4(m0 == 0 ? gv.x : 0.f, m0 == 1 ? gv.x : 0.f, m1 == 0 ? gv.y : 0.f, m1 == 1 ? gv.y : 0.f);
    const float4 b = make_float4(m0 == 2 ? gv.x : 0.f, m0 == 3 ? gv.x : 0.f, m1 == 2 ? gv.y : 0.f, m1 == 3 ? gv.y : 0.f);
    float4* p = reinterpret_cast<float4*>(dx + (row * 2) * w) + xo;
    p[0] = a;
    p[w >> 2] = b;
  }
}
__global__ void __launch_bounds__(kThreads) pool_bwd_2x2_from_output_scalar(const float* __restrict__ y, const float* __restrict__ g,
                                                                             const float* __restrict__ idx, float* __restrict__ dx,
                                                                             int64_t total, int w, int wo) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
    const int xo = (int)(o % wo);
    const int64_t row = o / wo;
    const float gv = __ldg(y + o) > 0.f ? __ldg(g + o) : 0.f;
    const int mi = (int)lrintf(__ldg(idx + o));
    float* p = dx + (row * 2) * w + 2 * xo;
    p[0] = mi == 0 ? gv : 0.f;
    p[1] = mi == 1 ? gv : 0.f;
    p[w] = mi == 2 ? gv : 0.f;
    p[w + 1] = mi == 3 ? gv : 0.f;
  }
}

// Disjoint windows: every input element is the target of at most one window, plain read-modify-write into a zero-filled dx.
__global__ void __launch_bounds__(kThreads) pool_bwd_general(const float* __restrict__ g, const float* __restrict__ idx,
                                                              float* __restrict__ dx, int64_t total, int h, int w, int ho,
                                                              int wo, int kw, int sh, int sw, int ph, int pw) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
    int xo = (int)(o % wo);
    int64_t r = o / wo;
    int yo = (int)(r % ho);
    int64_t bc = r / ho;
    long flat = lrintf(__ldg(idx + o));  // `.round() as usize` in the reference
    if (flat < 0) flat = 0;
    int ky = (int)(flat / kw), kx = (int)(flat % kw);
    int iy = yo * sh + ky - ph, ix = xo * sw + kx - pw;
    if (iy >= 0 && iy < h && ix >= 0 && ix < w) dx[(bc * h + iy) * w + ix] += __ldg(g + o);
  }
}

// Overlapping windows (stride < kernel): a thread per INPUT element visits the windows that cover it in ascending
// (yo, xo) order and adds the gradients of those whose saved index points at it.  No atomics and no zero-fill, and the
// order of the additions is the one of the reference's sequential scatter, so the result is reproducible bit for bit.
__global__ void __launch_bounds__(kThreads) pool_bwd_gather(const float* __restrict__ g, const float* __restrict__ idx,
                                                             float* __restrict__ dx, int64_t in_total, int h, int w, int ho,
                                                             int wo, int kh, int kw, int sh, int sw, int ph, int pw) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < in_total; e += stride) {
    const int ix = (int)(e % w);
    const int64_t r = e / w;
    const int iy = (int)(r % h);
    const int64_t bc = r / h;
    const int ny = iy + ph - kh + 1, nx = ix + pw - kw + 1;
    const int y_lo = ny > 0 ? (ny + sh - 1) / sh : 0, x_lo = nx > 0 ? (nx + sw - 1) / sw : 0;
    const int y_hi = min((iy + ph) / sh, ho - 1), x_hi = min((ix + pw) / sw, wo - 1);
    float acc = 0.f;
    for (int yo = y_lo; yo <= y_hi; ++yo) {
      const int ky = iy + ph - yo * sh;
      for (int xo = x_lo; xo <= x_hi; ++xo) {
        const int kx = ix + pw - xo * sw;
        const int64_t o = (bc * ho + yo) * wo + xo;
        long flat = lrintf(__ldg(idx + o));
        if (flat < 0) flat = 0;
        if (flat == (long)ky * kw + kx) acc += __ldg(g + o);
      }
    }
    dx[e] = acc;
  }
}

}  // namespace

extern "C" {

static rt_status pool_dims(rt_ctx* ctx, int64_t h, int64_t w, int kh, int kw, int sh, int sw, int ph, int pw, int64_t* ho,
                           int64_t* wo) {
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "max_pool2d: kernel and stride must be positive, padding non-negative");
  if (h + 2 * ph < kh || w + 2 * pw < kw) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "max_pool2d: window larger than padded input");
  if (h >= (1 << 30) || w >= (1 << 30)) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "max_pool2d: image too large");
  *ho = (h + 2 * ph - kh) / sh + 1;
  *wo = (w + 2 * pw - kw) / sw + 1;
  return RT_OK;
}

static rt_status pool_forward(rt_ctx* ctx, bool relu, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, int kh, int kw,
                              int sh, int sw, int ph, int pw, float* y, float* idx) {
  RT_CHECK_CTX(ctx);
  int64_t ho, wo;
  rt_status st = pool_dims(ctx, h, w, kh, kw, sh, sw, ph, pw, &ho, &wo);
  if (st != RT_OK) return st;
  int64_t total = n * c * ho * wo;
  if (total == 0) return RT_OK;
  RT_CHECK_PTR(ctx, x);
  RT_CHECK_PTR(ctx, y);
  RT_CHECK_PTR(ctx, idx);
  int grid = rt_grid_for(ctx, total, kThreads * 2);
  bool fast = kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && (h % 2 == 0) && (w % 2 == 0) &&
              (reinterpret_cast<uintptr_t>(x) % 8 == 0);
  if (fast) {
    if (relu) pool_fwd_2x2<true><<<grid, kThreads, 0, ctx->stream>>>(x, y, idx, total, (int)w, (int)ho, (int)wo);
    else pool_fwd_2x2<false><<<grid, kThreads, 0, ctx->stream>>>(x, y, idx, total, (int)w, (int)ho, (int)wo);
  } else {
    if (relu) pool_fwd_general<true><<<grid, kThreads, 0, ctx->stream>>>(x, y, idx, total, (int)h, (int)w, (int)ho, (int)wo, kh, kw, sh, sw, ph, pw);
    else pool_fwd_general<false><<<grid, kThreads, 0, ctx->stream>>>(x, y, idx, total, (int)h, (int)w, (int)ho, (int)wo, kh, kw, sh, sw, ph, pw);
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_max_pool2d(rt_ctx* ctx, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, int kh, int kw, int sh,
                        int sw, int ph, int pw, float* y, float* idx) {
  return pool_forward(ctx, false, x, n, c, h, w, kh, kw, sh, sw, ph, pw, y, idx);
}

rt_status rt_relu_max_pool2d(rt_ctx* ctx, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, int kh, int kw, int sh,
                             int sw, int ph, int pw, float* y, float* idx) {
  return pool_forward(ctx, true, x, n, c, h, w, kh, kw, sh, sw, ph, pw, y, idx);
}

// x != nullptr: backward of the fused relu + max_pool2d (dx masked with x > 0)
static rt_status pool_backward(rt_ctx* ctx, const float* x, const float* g, const float* idx, int64_t n, int64_t c, int64_t h,
                               int64_t w, int kh, int kw, int sh, int sw, int ph, int pw, float* dx) {
  RT_CHECK_CTX(ctx);
  int64_t ho, wo;
  rt_status st = pool_dims(ctx, h, w, kh, kw, sh, sw, ph, pw, &ho, &wo);
  if (st != RT_OK) return st;
  int64_t total = n * c * ho * wo, in_total = n * c * h * w;
  if (in_total == 0) return RT_OK;
  RT_CHECK_PTR(ctx, dx);
  bool fast = kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && (h % 2 == 0) && (w % 2 == 0) &&
              (reinterpret_cast<uintptr_t>(dx) % 8 == 0);
  if (fast) {
    if (total == 0) return RT_OK;
    RT_CHECK_PTR(ctx, g);
    RT_CHECK_PTR(ctx, idx);
    const bool pair = w % 4 == 0 && rt_aligned16(dx) && (reinterpret_cast<uintptr_t>(g) % 8 == 0) &&
                      (reinterpret_cast<uintptr_t>(idx) % 8 == 0) && (!x || rt_aligned16(x));
    if (pair) {  // w % 4 == 0 makes wo even: two windows per thread
      // one pair per thread up to 64 waves of blocks (a thread per pair measured 8.3 us on [256,32,28,28], eight waves 8.7)
      const int grid = rt_grid_for(ctx, total / 2, kThreads, 64);
      if (x) pool_bwd_2x2_pair<true><<<grid, kThreads, 0, ctx->stream>>>(g, idx, x, dx, total / 2, (int)w, (int)(wo / 2));
      else pool_bwd_2x2_pair<false><<<grid, kThreads, 0, ctx->stream>>>(g, idx, nullptr, dx, total / 2, (int)w, (int)(wo / 2));
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    const int grid2 = rt_grid_for(ctx, total, kThreads * 2);
    if (x && reinterpret_cast<uintptr_t>(x) % 8 == 0) {
      pool_bwd_2x2<true><<<grid2, kThreads, 0, ctx->stream>>>(g, idx, x, dx, total, (int)w, (int)ho, (int)wo);
      RT_LAUNCHED(ctx);
      return RT_OK;
    }
    pool_bwd_2x2<false><<<grid2, kThreads, 0, ctx->stream>>>(g, idx, nullptr, dx, total, (int)w, (int)ho, (int)wo);
    RT_LAUNCHED(ctx);
    return x ? rt_unary_backward(ctx, RT_RELU, x, dx, dx, in_total, 0.f, 0.f) : RT_OK;
  }
  const bool overlap = sh < kh || sw < kw;
  if (overlap && total > 0) {
    RT_CHECK_PTR(ctx, g);
    RT_CHECK_PTR(ctx, idx);
    pool_bwd_gather<<<rt_grid_for(ctx, in_total, kThreads * 2), kThreads, 0, ctx->stream>>>(g, idx, dx, in_total, (int)h, (int)w, (int)ho,
                                                                                          (int)wo, kh, kw, sh, sw, ph, pw);
    RT_LAUNCHED(ctx);
  } else {
    st = rt_fill(ctx, dx, 0.f, in_total);
    if (st != RT_OK || total == 0) return st;
    RT_CHECK_PTR(ctx, g);
    RT_CHECK_PTR(ctx, idx);
    pool_bwd_general<<<rt_grid_for(ctx, total, kThreads * 2), kThreads, 0, ctx->stream>>>(g, idx, dx, total, (int)h, (int)w, (int)ho, (int)wo,
                                                                                        kw, sh, sw, ph, pw);
    RT_LAUNCHED(ctx);
  }
  return x ? rt_unary_backward(ctx, RT_RELU, x, dx, dx, in_total, 0.f, 0.f) : RT_OK;  // element-wise, safe in place
}

rt_status rt_relu_max_pool2x2_backward_from_output(rt_ctx* ctx, const float* y, const float* g, const float* idx, int64_t n, int64_t c,
                                                   int64_t h, int64_t w, float* dx) {
  RT_CHECK_CTX(ctx);
  if (n < 0 || c < 0 || h < 0 || w < 0 || (h & 1) || (w & 1))
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "relu_max_pool2x2_backward_from_output: the un-pooled extent %lld x %lld must be even", (long long)h,
            (long long)w);
  const int64_t total = n * c * (h / 2) * (w / 2);
  if (total == 0) return RT_OK;
  RT_CHECK_PTR(ctx, y);
  RT_CHECK_PTR(ctx, g);
  RT_CHECK_PTR(ctx, idx);
  RT_CHECK_PTR(ctx, dx);
  const bool pair = w % 4 == 0 && rt_aligned16(dx) && (reinterpret_cast<uintptr_t>(g) % 8 == 0) && (reinterpret_cast<uintptr_t>(idx) % 8 == 0) &&
                    (reinterpret_cast<uintptr_t>(y) % 8 == 0);
  if (pair)
    pool_bwd_2x2_from_output<<<rt_grid_for(ctx, total / 2, kThreads, 64), kThreads, 0, ctx->stream>>>(y, g, idx, dx, total / 2, (int)w, (int)(w / 4));
  else
    pool_bwd_2x2_from_output_scalar<<<rt_grid_for(ctx, total, kThreads, 16), kThreads, 0, ctx->stream>>>(y, g, idx, dx, total, (int)w, (int)(w / 2));
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_max_pool2d_backward(rt_ctx* ctx, const float* g, const float* idx, int64_t n, int64_t c, int64_t h, int64_t w,
                                 int kh, int kw, int sh, int sw, int ph, int pw, float* dx) {
  return pool_backward(ctx, nullptr, g, idx, n, c, h, w, kh, kw, sh, sw, ph, pw, dx);
}

rt_status rt_relu_max_pool2d_backward(rt_ctx* ctx, const float* x, const float* g, const float* idx, int64_t n, int64_t c,
                                      int64_t h, int64_t w, int kh, int kw, int sh, int sw, int ph, int pw, float* dx) {
  RT_CHECK_CTX(ctx);
  if (n * c * h * w > 0) RT_CHECK_PTR(ctx, x);
  return pool_backward(ctx, x, g, idx, n, c, h, w, kh, kw, sh, sw, ph, pw, dx);
}

}  // extern "C"
