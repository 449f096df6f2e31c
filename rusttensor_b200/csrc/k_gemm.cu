// Dense contractions on the FP32 pipe: matmul (NN / NT / TN) and the implicit-GEMM
// forms of conv2d / conv2d_transpose and their gradients.  No im2col / col2im
// buffer is ever materialised: the operand tiles are gathered straight from the
// NCHW tensors while they are staged into shared memory.
//
// One register-blocked, double-buffered tile kernel serves every contraction; the
// operands are described by small loader functors (`load(row, k)`), the output by
// a store functor.  Products whose output is small but whose reduction is long
// (weight gradients) are split along K over blockIdx.z; the partial tiles are
// summed by a second, deterministic pass.
//
// This file is the exact-FP32 path.  Large, tile-aligned shapes are routed to the
// tcgen05 3xTF32 kernels in k_gemm_tc.cu by the dispatchers at the bottom.
#include "rt_internal.cuh"
#include "conv_geom.cuh"

rt_status rt_sum_axis_internal(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out,
                               float scale);
rt_status rt_gemm_tc_internal(rt_ctx* ctx, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, const float* a,
                              int64_t lda, const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate);

rt_status rt_conv_forward_tc_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g,
                                      float* y);
rt_status rt_conv_gather_tc_internal(rt_ctx* ctx, const float* y, const float* w, const float* bias, const ConvGeom& g,
                                     int cm, float* out);
rt_status rt_conv_weight_grad_tc_internal(rt_ctx* ctx, const float* x, const float* y, const ConvGeom& g, float* dw);
rt_status rt_conv_dw_tma_internal(rt_ctx* ctx, const float* x, const float* y, const ConvGeom& g, float* dw, float* db);
rt_status rt_conv_forward_thin_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g,
                                        float* y);
rt_status rt_conv_weight_grad_thin_internal(rt_ctx* ctx, const float* x, const float* gy, const ConvGeom& g, float* dw, float* db,
                                            bool* db_done);
rt_status rt_conv_relu_pool_thin_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g, float* y,
                                          float* idx);
rt_status rt_conv_window_tc_internal(rt_ctx* ctx, const float* src, int Nb, int C, int H, int W, int ph, int pw, const float* w,
                                     int N, int kh, int kw, int sn, int sc, int sky, int skx, int off0, const float* bias,
                                     float* out);

namespace {

// ---- operand loaders ---------------------------------------------------------------
// A-side loaders implement load(m, k); B-side loaders implement load(k, n).
// kContigK tells the tile loader which index runs fastest in memory, so that
// consecutive threads read consecutive addresses.

template <bool TRANS>  // A stored [M,K] (TRANS=false) or [K,M] (TRANS=true)
struct MatA {
  static constexpr bool kContigK = !TRANS;
  const float* p;
  int64_t ld;
  __device__ __forceinline__ float load(int m, int k) const { return TRANS ? __ldg(p + (int64_t)k * ld + m) : __ldg(p + (int64_t)m * ld + k); }
};
template <bool TRANS>  // B stored [K,N] (TRANS=false) or [N,K] (TRANS=true)
struct MatB {
  static constexpr bool kContigK = TRANS;
  const float* p;
  int64_t ld;
  __device__ __forceinline__ float load(int k, int n) const { return TRANS ? __ldg(p + (int64_t)n * ld + k) : __ldg(p + (int64_t)k * ld + n); }
};

// im2col view of X: rows k = (cx,ky,kx), columns n = (b,yo,xo).  Used as the B operand
// of the forward convolution.
struct Im2colB {
  static constexpr bool kContigK = false;
  const float* x;
  ConvGeom g;
  __device__ __forceinline__ float load(int k, int n) const {
    uint32_t cx, r, ky, kx, b, p, yo, xo;
    g.d_khw.divmod(k, cx, r);
    g.d_kw.divmod(r, ky, kx);
    g.d_HyWy.divmod(n, b, p);
    g.d_Wy.divmod(p, yo, xo);
    int iy = (int)(yo * g.sh + ky) - g.ph, ix = (int)(xo * g.sw + kx) - g.pw;
    if (iy < 0 || iy >= g.Hx || ix < 0 || ix >= g.Wx) return 0.f;
    return __ldg(x + (((int64_t)b * g.Cx + cx) * g.Hx + iy) * g.Wx + ix);
  }
};

// Same im2col view, transposed roles for the weight gradient: reduction index
// k = (b,yo,xo), columns n = (cx,ky,kx).
struct Im2colK {
  static constexpr bool kContigK = true;
  const float* x;
  ConvGeom g;
  __device__ __forceinline__ float load(int k, int n) const {
    uint32_t cx, r, ky, kx, b, p, yo, xo;
    g.d_khw.divmod(n, cx, r);
    g.d_kw.divmod(r, ky, kx);
    g.d_HyWy.divmod(k, b, p);
    g.d_Wy.divmod(p, yo, xo);
    int iy = (int)(yo * g.sh + ky) - g.ph, ix = (int)(xo * g.sw + kx) - g.pw;
    if (iy < 0 || iy >= g.Hx || ix < 0 || ix >= g.Wx) return 0.f;
    return __ldg(x + (((int64_t)b * g.Cx + cx) * g.Hx + iy) * g.Wx + ix);
  }
};

// Y as the A operand of the weight gradient: rows m = cy, reduction k = (b,yo,xo).
struct NarrowA {
  static constexpr bool kContigK = true;
  const float* y;
  ConvGeom g;
  __device__ __forceinline__ float load(int m, int k) const {
    uint32_t b, p;
    g.d_HyWy.divmod(k, b, p);
    return __ldg(y + ((int64_t)b * g.Cy + m) * (g.Hy * g.Wy) + p);
  }
};

// Weights [Cred, Cm, kh, kw] read as A(m, k) with k = (cred, ky, kx): the operand of
// the input-gradient / transposed-convolution gather.
struct WeightSecondIndexA {
  static constexpr bool kContigK = true;
  const float* w;
  int Cm;
  ConvGeom g;
  __device__ __forceinline__ float load(int m, int k) const {
    uint32_t cr, r;
    g.d_khw.divmod(k, cr, r);
    return __ldg(w + ((int64_t)cr * Cm + m) * (g.kh * g.kw) + r);
  }
};

// Gather view of Y for the input gradient: rows k = (cy,ky,kx), columns n = (b,iy,ix);
// element = y(b,cy,(iy+ph-ky)/sh,(ix+pw-kx)/sw) when the division is exact and in range.
struct GatherB {
  static constexpr bool kContigK = false;
  const float* y;
  ConvGeom g;
  __device__ __forceinline__ float load(int k, int n) const {
    uint32_t cy, r, ky, kx, b, p, iy, ix;
    g.d_khw.divmod(k, cy, r);
    g.d_kw.divmod(r, ky, kx);
    g.d_HxWx.divmod(n, b, p);
    g.d_Wx.divmod(p, iy, ix);
    int ty = (int)iy + g.ph - (int)ky, tx = (int)ix + g.pw - (int)kx;
    if (ty < 0 || tx < 0) return 0.f;
    uint32_t yo, ry, xo, rx;
    g.d_sh.divmod(ty, yo, ry);
    g.d_sw.divmod(tx, xo, rx);
    if (ry != 0 || rx != 0 || (int)yo >= g.Hy || (int)xo >= g.Wy) return 0.f;
    return __ldg(y + (((int64_t)b * g.Cy + cy) * g.Hy + yo) * g.Wy + xo);
  }
};

// ---- output stores -------------------------------------------------------------------
struct PlainC {  // C[(z*M + m)*ld + n]; z = split index (0 when not split)
  float* c;
  int64_t ld;
  int64_t split_stride;
  bool accumulate;
  __device__ __forceinline__ void store(int m, int n, float v, int z) const {
    float* q = c + z * split_stride + (int64_t)m * ld + n;
    *q = accumulate ? *q + v : v;
  }
};
struct ImageC {  // out[b, m, p] with n = (b,p), optional per-channel bias
  float* out;
  const float* bias;
  int C;
  int HW;
  FastDiv d_HW;
  __device__ __forceinline__ void store(int m, int n, float v, int) const {
    uint32_t b, p;
    d_HW.divmod(n, b, p);
    out[((int64_t)b * C + m) * HW + p] = bias ? v + __ldg(bias + m) : v;
  }
};

// ---- the tile kernel -------------------------------------------------------------------
constexpr int BK = 16;

template <int BM, int BN, int TM, int TN, class LA, class LB, class SC>
__global__ void __launch_bounds__(256) gemm_tile_kernel(LA la, LB lb, SC sc, int M, int N, int K, int k_per_split) {
  static_assert((BM / TM) * (BN / TN) == 256, "256 threads per tile");
  static_assert(TM % 4 == 0 && TN % 4 == 0, "register tile is made of 4-wide groups");
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  constexpr int TX = BN / TN;
  constexpr int GM = TM / 4, GN = TN / 4;            // 4-wide groups per thread
  constexpr int SM_ = BM / GM, SN_ = BN / GN;        // spacing between groups
  constexpr int NA = BM * BK / 256, NB = BN * BK / 256;
  const int t = threadIdx.x;
  const int tx = t % TX, ty = t / TX;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kbeg = blockIdx.z * k_per_split;
  const int kend = min(K, kbeg + k_per_split);

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  float ra[NA], rb[NB];

  auto gload = [&](int k0) {
#pragma unroll
    for (int i = 0; i < NA; ++i) {
      int e = t + i * 256;
      int kk = LA::kContigK ? e % BK : e / BM;
      int mm = LA::kContigK ? e / BK : e % BM;
      int m = m0 + mm, k = k0 + kk;
      ra[i] = (m < M && k < kend) ? la.load(m, k) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      int e = t + i * 256;
      int kk = LB::kContigK ? e % BK : e / BN;
      int nn = LB::kContigK ? e / BK : e % BN;
      int n = n0 + nn, k = k0 + kk;
      rb[i] = (n < N && k < kend) ? lb.load(k, n) : 0.f;
    }
  };
  auto sstore = [&](int buf) {
#pragma unroll
    for (int i = 0; i < NA; ++i) {
      int e = t + i * 256;
      int kk = LA::kContigK ? e % BK : e / BM;
      int mm = LA::kContigK ? e / BK : e % BM;
      As[buf][kk][mm] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      int e = t + i * 256;
      int kk = LB::kContigK ? e % BK : e / BN;
      int nn = LB::kContigK ? e / BK : e % BN;
      Bs[buf][kk][nn] = rb[i];
    }
  };

  if (kbeg < kend) {
    gload(kbeg);
    sstore(0);
  }
  __syncthreads();
  int buf = 0;
  for (int k0 = kbeg; k0 < kend; k0 += BK) {
    const bool has_next = k0 + BK < kend;
    if (has_next) gload(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int gi = 0; gi < GM; ++gi) {
        float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][gi * SM_ + ty * 4]);
        a[gi * 4 + 0] = v.x; a[gi * 4 + 1] = v.y; a[gi * 4 + 2] = v.z; a[gi * 4 + 3] = v.w;
      }
#pragma unroll
      for (int gj = 0; gj < GN; ++gj) {
        float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][gj * SN_ + tx * 4]);
        b[gj * 4 + 0] = v.x; b[gj * 4 + 1] = v.y; b[gj * 4 + 2] = v.z; b[gj * 4 + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (has_next) sstore(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + (i / 4) * SM_ + ty * 4 + (i % 4);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int n = n0 + (j / 4) * SN_ + tx * 4 + (j % 4);
      if (n < N) sc.store(m, n, acc[i][j], blockIdx.z);
    }
  }
}

template <int BM, int BN, int TM, int TN, class LA, class LB, class SC>
void launch_tile(rt_ctx* ctx, const LA& la, const LB& lb, const SC& sc, int M, int N, int K, int splits, int kps) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
  gemm_tile_kernel<BM, BN, TM, TN, LA, LB, SC><<<grid, 256, 0, ctx->stream>>>(la, lb, sc, M, N, K, kps);
}

// Picks a tile shape for (M, N) and launches.  splits > 1 requires a PlainC store that
// points at a [splits, M, N] workspace.
template <class LA, class LB, class SC>
rt_status run_gemm(rt_ctx* ctx, const LA& la, const LB& lb, const SC& sc, int64_t M, int64_t N, int64_t K, int splits,
                   int kps) {
  if (M <= 0 || N <= 0) return RT_OK;
  if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31))
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "contraction extent exceeds 2^31");
  if (M <= 32) launch_tile<32, 128, 4, 4>(ctx, la, lb, sc, (int)M, (int)N, (int)K, splits, kps);
  else if (N <= 32) launch_tile<128, 32, 4, 4>(ctx, la, lb, sc, (int)M, (int)N, (int)K, splits, kps);
  else if (M <= 64 || N <= 64) launch_tile<64, 64, 4, 4>(ctx, la, lb, sc, (int)M, (int)N, (int)K, splits, kps);
  else launch_tile<128, 128, 8, 8>(ctx, la, lb, sc, (int)M, (int)N, (int)K, splits, kps);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

int tiles_for(int64_t M, int64_t N) {
  int bm, bn;
  if (M <= 32) { bm = 32; bn = 128; }
  else if (N <= 32) { bm = 128; bn = 32; }
  else if (M <= 64 || N <= 64) { bm = 64; bn = 64; }
  else { bm = 128; bn = 128; }
  return (int)(((M + bm - 1) / bm) * ((N + bn - 1) / bn));
}

// Split-K policy: fill about two waves of SMs, keep at least 256 reduction steps per split.
void choose_split(rt_ctx* ctx, int64_t M, int64_t N, int64_t K, int* splits, int* kps) {
  int tiles = tiles_for(M, N);
  int64_t want = ((int64_t)ctx->sm_count * 2 + tiles - 1) / tiles;
  int64_t max_s = K / 256;
  if (max_s < 1) max_s = 1;
  int64_t s = want < max_s ? want : max_s;
  if (s < 1) s = 1;
  if (s > 1024) s = 1024;
  int64_t per = (K + s - 1) / s;
  per = (per + BK - 1) / BK * BK;
  s = (K + per - 1) / per;
  if (s < 1) s = 1;
  *splits = (int)s;
  *kps = (int)per;
}

// C[M,N] (row-major, ld == N when split) = A x B with optional split-K.
template <class LA, class LB>
rt_status gemm_plain(rt_ctx* ctx, const LA& la, const LB& lb, float* c, int64_t ldc, int64_t M, int64_t N, int64_t K,
                     bool accumulate, bool allow_split) {
  if (M <= 0 || N <= 0) return RT_OK;
  if (K <= 0) {
    if (accumulate) return RT_OK;
    if (ldc == N) return rt_fill(ctx, c, 0.f, M * N);
    for (int64_t m = 0; m < M; ++m) {
      rt_status st = rt_fill(ctx, c + m * ldc, 0.f, N);
      if (st != RT_OK) return st;
    }
    return RT_OK;
  }
  int splits = 1, kps = (int)((K + BK - 1) / BK * BK);
  if (allow_split && !accumulate && ldc == N) choose_split(ctx, M, N, K, &splits, &kps);
  if (splits == 1) {
    PlainC sc{c, ldc, 0, accumulate};
    return run_gemm(ctx, la, lb, sc, M, N, K, 1, kps);
  }
  RtScratch ws(ctx);
  rt_status st = ws.alloc(sizeof(float) * (size_t)splits * M * N);
  if (st != RT_OK) return st;
  PlainC sc{ws.as<float>(), N, M * N, false};
  st = run_gemm(ctx, la, lb, sc, M, N, K, splits, kps);
  if (st != RT_OK) return st;
  return rt_sum_axis_internal(ctx, ws.as<float>(), 1, splits, M * N, c, 1.f);
}

// ---- narrow products -------------------------------------------------------------------------------------------
// A classifier head (N <= 16 output columns) or its input gradient (K <= 16) gives a tile kernel one or two CTAs that
// walk K serially; these two kernels spread the same arithmetic over the block instead.
constexpr int kSkinnyN = 16, kSkinnyRows = 32, kSkinnyKC = 128, kSkinnySlices = 8;

// C[M, N<=16] = A x B.  A block owns 32 rows of C: A and B chunks of 128 k are staged in shared memory with coalesced
// loads whatever the storage order, thread (row, slice) accumulates every 8th k, the 8 slices are added in a fixed order.
template <bool TA, bool TB>
__global__ void __launch_bounds__(kSkinnyRows * kSkinnySlices)
gemm_skinny_n_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ b, int64_t ldb, float* __restrict__ c,
                     int64_t ldc, int M, int N, int K, int accumulate) {
  constexpr int T = kSkinnyRows * kSkinnySlices;
  __shared__ float As[kSkinnyRows][kSkinnyKC + 1];
  __shared__ __align__(16) float Bs[kSkinnyKC][kSkinnyN];
  __shared__ float red[kSkinnySlices][kSkinnyRows][kSkinnyN + 1];
  const int tid = threadIdx.x, ml = tid & 31, ks = tid >> 5;
  const int m0 = blockIdx.x * kSkinnyRows;
  float acc[kSkinnyN];
#pragma unroll
  for (int j = 0; j < kSkinnyN; ++j) acc[j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kSkinnyKC) {
    // all loads of the chunk are issued before the first store, so the chunk costs one memory round trip
    constexpr int kALoads = kSkinnyRows * kSkinnyKC / T, kBLoads = kSkinnyKC * kSkinnyN / T;
    float ar[kALoads], br_[kBLoads];
#pragma unroll
    for (int u = 0; u < kALoads; ++u) {
      const int i = tid + u * T;
      int mm, kk;
      if (TA) { mm = i % kSkinnyRows; kk = i / kSkinnyRows; } else { kk = i % kSkinnyKC; mm = i / kSkinnyKC; }
      const bool in = m0 + mm < M && k0 + kk < K;
      const int64_t off = TA ? (int64_t)(k0 + kk) * lda + m0 + mm : (int64_t)(m0 + mm) * lda + k0 + kk;
      ar[u] = in ? __ldg(a + off) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kBLoads; ++u) {
      const int i = tid + u * T;
      int j, kk;
      if (TB) { kk = i % kSkinnyKC; j = i / kSkinnyKC; } else { j = i % kSkinnyN; kk = i / kSkinnyN; }
      const bool in = j < N && k0 + kk < K;
      const int64_t off = TB ? (int64_t)j * ldb + k0 + kk : (int64_t)(k0 + kk) * ldb + j;
      br_[u] = in ? __ldg(b + off) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kALoads; ++u) {
      const int i = tid + u * T;
      if (TA) As[i % kSkinnyRows][i / kSkinnyRows] = ar[u]; else As[i / kSkinnyKC][i % kSkinnyKC] = ar[u];
    }
#pragma unroll
    for (int u = 0; u < kBLoads; ++u) {
      const int i = tid + u * T;
      if (TB) Bs[i % kSkinnyKC][i / kSkinnyKC] = br_[u]; else Bs[i / kSkinnyN][i % kSkinnyN] = br_[u];
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = ks; kk < kSkinnyKC; kk += kSkinnySlices) {
      const float av = As[ml][kk];
      const float4* br = reinterpret_cast<const float4*>(&Bs[kk][0]);
#pragma unroll
      for (int q = 0; q < kSkinnyN / 4; ++q) {
        const float4 bv = br[q];
        acc[q * 4 + 0] = fmaf(av, bv.x, acc[q * 4 + 0]);
        acc[q * 4 + 1] = fmaf(av, bv.y, acc[q * 4 + 1]);
        acc[q * 4 + 2] = fmaf(av, bv.z, acc[q * 4 + 2]);
        acc[q * 4 + 3] = fmaf(av, bv.w, acc[q * 4 + 3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < kSkinnyN; ++j) red[ks][ml][j] = acc[j];
  __syncthreads();
  for (int o = tid; o < kSkinnyRows * kSkinnyN; o += T) {
    const int mm = o / kSkinnyN, j = o % kSkinnyN;
    if (m0 + mm >= M || j >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kSkinnySlices; ++s2) v += red[s2][mm][j];
    float* dst = c + (int64_t)(m0 + mm) * ldc + j;
    *dst = accumulate ? *dst + v : v;
  }
}

// C[M, N] = A x B for K <= 16: one thread per output element, B (K x N, a few KB) read through the cache.
template <bool TA, bool TB>
__global__ void __launch_bounds__(256) gemm_small_k_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ b,
                                                           int64_t ldb, float* __restrict__ c, int64_t ldc, int64_t MN, int N, int K,
                                                           int accumulate) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < MN; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = e / N;
    const int j = (int)(e - i * N);
    float av[16], bv[16];
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      av[kk] = kk < K ? __ldg(a + (TA ? (int64_t)kk * lda + i : i * lda + kk)) : 0.f;
      bv[kk] = kk < K ? __ldg(b + (TB ? (int64_t)j * ldb + kk : (int64_t)kk * ldb + j)) : 0.f;
    }
    float v = 0.f;
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) v = fmaf(av[kk], bv[kk], v);
    float* dst = c + i * ldc + j;
    *dst = accumulate ? *dst + v : v;
  }
}

template <bool TA, bool TB>
rt_status gemm_narrow_launch(rt_ctx* ctx, int64_t m, int64_t n, int64_t k, const float* a, int64_t lda, const float* b,
                             int64_t ldb, float* c, int64_t ldc, int accumulate) {
  if (k <= 16) {
    gemm_small_k_kernel<TA, TB><<<rt_grid_for(ctx, m * n, 256), 256, 0, ctx->stream>>>(a, lda, b, ldb, c, ldc, m * n, (int)n,
                                                                                      (int)k, accumulate);
  } else {
    const int grid = (int)((m + kSkinnyRows - 1) / kSkinnyRows);
    gemm_skinny_n_kernel<TA, TB><<<grid, kSkinnyRows * kSkinnySlices, 0, ctx->stream>>>(a, lda, b, ldb, c, ldc, (int)m, (int)n,
                                                                                        (int)k, accumulate);
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// Narrow products (K <= 16, or N <= 16 with a K one block can walk); RT_ERR_UNIMPLEMENTED for everything else.
rt_status gemm_narrow(rt_ctx* ctx, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, const float* a, int64_t lda,
                      const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate) {
  if (k < 1 || m >= (1ll << 31) || n >= (1ll << 31) || m * n >= (1ll << 40)) return RT_ERR_UNIMPLEMENTED;
  const bool small_k = k <= 16;
  const bool skinny_n = n <= kSkinnyN && (k <= 4096 || m >= 4096) && k < (1ll << 30) && m < (1ll << 30);
  if (!small_k && !skinny_n) return RT_ERR_UNIMPLEMENTED;
  if (!trans_a && !trans_b) return gemm_narrow_launch<false, false>(ctx, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
  if (!trans_a && trans_b) return gemm_narrow_launch<false, true>(ctx, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
  if (trans_a && !trans_b) return gemm_narrow_launch<true, false>(ctx, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
  return gemm_narrow_launch<true, true>(ctx, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
}

rt_status check_conv_args(rt_ctx* ctx, int64_t n, int64_t cin, int64_t h, int64_t w, int64_t cout, int kh, int kw, int sh,
                          int sw, int ph, int pw) {
  if (n < 0 || cin < 0 || h < 0 || w < 0 || cout < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "conv: negative extent");
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv: kernel and stride must be positive, padding non-negative");
  return RT_OK;
}

// y[Nb,Cy,Hy,Wy] = conv(x[Nb,Cx,Hx,Wx], w[Cy,Cx,kh,kw]) (+bias)
rt_status conv_forward_like(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g, float* y) {
  int64_t M = g.Cy, N = (int64_t)g.Nb * g.Hy * g.Wy, K = (int64_t)g.Cx * g.kh * g.kw;
  if (M == 0 || N == 0) return RT_OK;
  if (ctx->use_tensor_cores) {  // tiny reductions: direct FP32 kernel
    rt_status st = rt_conv_forward_thin_internal(ctx, x, w, bias, g, y);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores && g.sh == 1 && g.sw == 1) {
    rt_status st = rt_conv_window_tc_internal(ctx, x, g.Nb, g.Cx, g.Hx, g.Wx, g.ph, g.pw, w, g.Cy, g.kh, g.kw, g.Cx * g.kh * g.kw,
                                              g.kh * g.kw, g.kw, 1, 0, bias, y);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores) {
    rt_status st = rt_conv_forward_tc_internal(ctx, x, w, bias, g, y);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  MatA<false> la{w, K};
  Im2colB lb{x, g};
  ImageC sc{y, bias, g.Cy, g.Hy * g.Wy, {}};
  sc.d_HW.init(g.Hy * g.Wy);
  return run_gemm(ctx, la, lb, sc, M, N, K, 1, (int)((K + BK - 1) / BK * BK));
}

// dw[Cy, Cx*kh*kw] = sum over (b,yo,xo) of y * im2col(x)
// With `db` not null the bias gradient db[Cy] = sum over (b, pixels) of y may be produced in the same pass; *db_done
// tells whether it was.
rt_status conv_weight_grad_like(rt_ctx* ctx, const float* x, const float* y, const ConvGeom& g, float* dw, float* db = nullptr,
                                bool* db_done = nullptr) {
  int64_t M = g.Cy, N = (int64_t)g.Cx * g.kh * g.kw, K = (int64_t)g.Nb * g.Hy * g.Wy;
  if (db_done) *db_done = false;
  if (ctx->use_tensor_cores && ctx->use_tma_weight_grad && M > 0 && N > 0 && K > 0) {  // unit stride: TMA-fed, pixels as K
    rt_status st = rt_conv_dw_tma_internal(ctx, x, y, g, dw, db);
    if (st == RT_OK && db && db_done) *db_done = true;
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores && M > 0 && N > 0 && K > 0) {  // tiny reductions: direct FP32 kernel
    rt_status st = rt_conv_weight_grad_thin_internal(ctx, x, y, g, dw, db, db_done);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores && M > 0 && N > 0) {
    rt_status st = rt_conv_weight_grad_tc_internal(ctx, x, y, g, dw);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  NarrowA la{y, g};
  Im2colK lb{x, g};
  return gemm_plain(ctx, la, lb, dw, N, M, N, K, false, true);
}

// out[Nb,Cm,Hx,Wx] (+bias) = gather of y[Nb,Cy,Hy,Wy] with w[Cy,Cm,kh,kw]
rt_status conv_gather_like(rt_ctx* ctx, const float* y, const float* w, const float* bias, const ConvGeom& g, int cm,
                           float* out) {
  int64_t M = cm, N = (int64_t)g.Nb * g.Hx * g.Wx, K = (int64_t)g.Cy * g.kh * g.kw;
  if (M == 0 || N == 0) return RT_OK;
  if (ctx->use_tensor_cores && g.sh == 1 && g.sw == 1) {
    // unit stride: a convolution of y with the kernel flipped in both directions and padding (kh-1-ph, kw-1-pw)
    rt_status st = rt_conv_window_tc_internal(ctx, y, g.Nb, g.Cy, g.Hy, g.Wy, g.kh - 1 - g.ph, g.kw - 1 - g.pw, w, cm, g.kh, g.kw,
                                              g.kh * g.kw, cm * g.kh * g.kw, -g.kw, -1, g.kh * g.kw - 1, bias, out);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores) {
    rt_status st = rt_conv_gather_tc_internal(ctx, y, w, bias, g, cm, out);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  WeightSecondIndexA la{w, cm, g};
  GatherB lb{y, g};
  ImageC sc{out, bias, cm, g.Hx * g.Wx, {}};
  sc.d_HW.init(g.Hx * g.Wx);
  return run_gemm(ctx, la, lb, sc, M, N, K, 1, (int)((K + BK - 1) / BK * BK));
}

// db[c] = sum over batch and pixels of t[Nb, C, HW]
rt_status channel_sum(rt_ctx* ctx, const float* t, int64_t nb, int64_t c, int64_t hw, float* db) {
  if (c == 0) return RT_OK;
  if (nb == 0 || hw == 0) return rt_fill(ctx, db, 0.f, c);
  RtScratch tmp(ctx);
  rt_status st = tmp.alloc(sizeof(float) * nb * c);
  if (st != RT_OK) return st;
  st = rt_sum_axis_internal(ctx, t, nb * c, hw, 1, tmp.as<float>(), 1.f);
  if (st != RT_OK) return st;
  return rt_sum_axis_internal(ctx, tmp.as<float>(), 1, nb, c, db, 1.f);
}

}  // namespace

extern "C" {

rt_status rt_gemm(rt_ctx* ctx, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, const float* a, int64_t lda,
                  const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate) {
  RT_CHECK_CTX(ctx);
  if (m < 0 || n < 0 || k < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_gemm: negative extent");
  if (m == 0 || n == 0) return RT_OK;
  RT_CHECK_PTR(ctx, c);
  if (k > 0) {
    RT_CHECK_PTR(ctx, a);
    RT_CHECK_PTR(ctx, b);
  }
  if (lda < (trans_a ? m : k) || ldb < (trans_b ? k : n) || ldc < n)
    RT_FAIL(ctx, RT_ERR_SHAPE_MISMATCH, "rt_gemm: leading dimension smaller than the row length");
  bool acc = accumulate != 0;
  if (ctx->use_tensor_cores) {  // narrow products: dedicated FP32 kernels
    rt_status st = gemm_narrow(ctx, trans_a, trans_b, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (ctx->use_tensor_cores && k >= 32 && m >= 32 && n >= 16 && m * n * k >= (1ll << 20)) {
    rt_status st = rt_gemm_tc_internal(ctx, trans_a, trans_b, m, n, k, a, lda, b, ldb, c, ldc, accumulate);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  if (!trans_a && !trans_b) return gemm_plain(ctx, MatA<false>{a, lda}, MatB<false>{b, ldb}, c, ldc, m, n, k, acc, true);
  if (!trans_a && trans_b) return gemm_plain(ctx, MatA<false>{a, lda}, MatB<true>{b, ldb}, c, ldc, m, n, k, acc, true);
  if (trans_a && !trans_b) return gemm_plain(ctx, MatA<true>{a, lda}, MatB<false>{b, ldb}, c, ldc, m, n, k, acc, true);
  return gemm_plain(ctx, MatA<true>{a, lda}, MatB<true>{b, ldb}, c, ldc, m, n, k, acc, true);
}

static rt_status matmul_backward_impl(rt_ctx* ctx, const float* a, const float* b, const float* g, int64_t m, int64_t k, int64_t n,
                                      float* da, float* db, int accumulate_db) {
  RT_CHECK_CTX(ctx);
  // da[M,K] = g[M,N] * b[K,N]^T ; db[K,N] (+)= a[M,K]^T * g[M,N]: independent, so db goes to the side stream
  RtFork fork(ctx, da && db);
  rt_status st = RT_OK, st2 = RT_OK;
  if (db) st2 = rt_gemm(ctx, 1, 0, k, n, m, a, k, g, n, db, n, accumulate_db);
  rt_status e1 = fork.end();
  if (da) st = rt_gemm(ctx, 0, 1, m, k, n, g, n, b, n, da, k, 0);
  rt_status e2 = fork.join();
  if (st != RT_OK) return st;
  if (st2 != RT_OK) return st2;
  return e1 != RT_OK ? e1 : e2;
}

rt_status rt_matmul_backward(rt_ctx* ctx, const float* a, const float* b, const float* g, int64_t m, int64_t k, int64_t n,
                             float* da, float* db) {
  return matmul_backward_impl(ctx, a, b, g, m, k, n, da, db, 0);
}

rt_status rt_matmul_backward_accumulate(rt_ctx* ctx, const float* a, const float* b, const float* g, int64_t m, int64_t k, int64_t n,
                                        float* da, float* db_sum) {
  return matmul_backward_impl(ctx, a, b, g, m, k, n, da, db_sum, 1);
}

rt_status rt_conv2d(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n, int64_t cin, int64_t h,
                    int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw, float* y) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_conv_args(ctx, n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if (st != RT_OK) return st;
  if (h + 2 * ph < kh || wd + 2 * pw < kw) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d: kernel larger than padded input");
  ConvGeom g = make_geom(n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if ((int64_t)n * cout * g.Hy * g.Wy == 0) return RT_OK;
  RT_CHECK_PTR(ctx, y);
  return conv_forward_like(ctx, x, w, bias, g, y);
}

rt_status rt_conv2d_relu_max_pool2x2(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n, int64_t cin, int64_t h,
                                     int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw, float* y, float* idx) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_conv_args(ctx, n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if (st != RT_OK) return st;
  if (h + 2 * ph < kh || wd + 2 * pw < kw) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d_relu_max_pool2x2: kernel larger than padded input");
  ConvGeom g = make_geom(n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if ((g.Hy & 1) || (g.Wy & 1))
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d_relu_max_pool2x2: the convolution output %d x %d must have even extents", g.Hy, g.Wy);
  if ((int64_t)n * cout * g.Hy * g.Wy == 0) return RT_OK;
  RT_CHECK_PTR(ctx, y);
  RT_CHECK_PTR(ctx, idx);
  if (ctx->use_tensor_cores) {  // the fused first-layer kernel (exact FP32, like the unfused first-layer kernel it mirrors)
    st = rt_conv_relu_pool_thin_internal(ctx, x, w, bias, g, y, idx);
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  // every other shape: the convolution into scratch memory, then relu + pooling in one kernel; the scratch block goes back to
  // the pool when this call returns
  RtScratch conv_out(ctx);
  st = conv_out.alloc(sizeof(float) * (size_t)n * cout * g.Hy * g.Wy);
  if (st != RT_OK) return st;
  st = conv_forward_like(ctx, x, w, bias, g, conv_out.as<float>());
  if (st != RT_OK) return st;
  return rt_relu_max_pool2d(ctx, conv_out.as<float>(), n, cout, g.Hy, g.Wy, 2, 2, 2, 2, 0, 0, y, idx);
}

rt_status rt_conv2d_backward(rt_ctx* ctx, const float* x, const float* w, const float* gr, int64_t n, int64_t cin,
                             int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw,
                             float* dx, float* dw, float* db) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_conv_args(ctx, n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if (st != RT_OK) return st;
  if (h + 2 * ph < kh || wd + 2 * pw < kw) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d_backward: kernel larger than padded input");
  ConvGeom g = make_geom(n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  // The three gradients are independent.  The bias gradient (bandwidth-bound, small footprint) goes to the side stream,
  // where it overlaps the contraction kernels.
  RtFork fork(ctx, db && (dw || dx));
  rt_status st_b = RT_OK;
  // The weight gradient goes to the side stream with the bias gradient (its kernel may produce the bias gradient in
  // the same pass over the upstream gradient); the input gradient stays on the main stream.
  bool db_done = false;
  if (dw) st = conv_weight_grad_like(ctx, x, gr, g, dw, db, &db_done);
  if (db && !db_done) st_b = channel_sum(ctx, gr, n, cout, (int64_t)g.Hy * g.Wy, db);
  rt_status e1 = fork.end();
  if (st == RT_OK && dx) {
    // positions never touched by a window (possible when stride > kernel) must read as 0:
    // the gather computes every dx element, so no pre-fill is needed.
    st = conv_gather_like(ctx, gr, w, nullptr, g, (int)cin, dx);
  }
  rt_status e2 = fork.join();
  if (st != RT_OK) return st;
  if (st_b != RT_OK) return st_b;
  return e1 != RT_OK ? e1 : e2;
}

rt_status rt_conv2d_transpose(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n, int64_t cin,
                              int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw,
                              float* y) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_conv_args(ctx, n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if (st != RT_OK) return st;
  if (h < 1 || wd < 1) return RT_OK;
  int64_t oh = (h - 1) * sh + kh - 2 * ph, ow = (wd - 1) * sw + kw - 2 * pw;
  if (oh <= 0 || ow <= 0) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d_transpose: empty output");
  // The transposed convolution is the gather of x through a convolution whose wide side is
  // the OUTPUT (oh x ow) and whose narrow side is the input (h x w).
  ConvGeom g = make_geom(n, cout, oh, ow, cin, kh, kw, sh, sw, ph, pw);
  if (g.Hy != h || g.Wy != wd) {
    // (oh + 2p - k) / s + 1 can exceed h when the division truncates; restrict to the real input.
    g.Hy = (int)h;
    g.Wy = (int)wd;
    g.finish();
  }
  return conv_gather_like(ctx, x, w, bias, g, (int)cout, y);
}

rt_status rt_conv2d_transpose_backward(rt_ctx* ctx, const float* x, const float* w, const float* gr, int64_t n,
                                       int64_t cin, int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw,
                                       int ph, int pw, float* dx, float* dw, float* db) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_conv_args(ctx, n, cin, h, wd, cout, kh, kw, sh, sw, ph, pw);
  if (st != RT_OK) return st;
  if (h < 1 || wd < 1) return RT_OK;
  int64_t oh = (h - 1) * sh + kh - 2 * ph, ow = (wd - 1) * sw + kw - 2 * pw;
  if (oh <= 0 || ow <= 0) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "conv2d_transpose_backward: empty output");
  // wide = grad_output [n, cout, oh, ow]; narrow = x [n, cin, h, w]
  ConvGeom g = make_geom(n, cout, oh, ow, cin, kh, kw, sh, sw, ph, pw);
  g.Hy = (int)h;
  g.Wy = (int)wd;
  g.finish();
  // as in rt_conv2d_backward: bias gradient (and the weight gradient, when dx is wanted too) on the side stream
  RtFork fork(ctx, db && (dw || dx));
  rt_status st_side = RT_OK;
  if (db) st_side = channel_sum(ctx, gr, n, cout, oh * ow, db);
  if (st_side == RT_OK && dw && dx && fork.open) {  // dw[cin, cout*kh*kw] = sum x * im2col(grad_output)
    st_side = conv_weight_grad_like(ctx, gr, x, g, dw);
    dw = nullptr;
  }
  rt_status e1 = fork.end();
  if (dx) st = conv_forward_like(ctx, gr, w, nullptr, g, dx);  // dx = conv(grad_output, w viewed as [cin, cout, kh, kw])
  if (st == RT_OK && dw) st = conv_weight_grad_like(ctx, gr, x, g, dw);
  rt_status e2 = fork.join();
  if (st != RT_OK) return st;
  if (st_side != RT_OK) return st_side;
  return e1 != RT_OK ? e1 : e2;
}

}  // extern "C"
