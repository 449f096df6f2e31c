// Dense contractions on the 5th-generation tensor cores (tcgen05) with 3xTF32 emulation
// of fp32: every fp32 operand is split as a = hi + lo (hi = a with the low 13 mantissa
// bits cleared, lo = a - hi, exact), and a*b is accumulated as hi*hi + hi*lo + lo*hi in an
// fp32 accumulator held in tensor memory (TMEM).  The dropped lo*lo term and the rounding
// of lo to TF32 are O(2^-21) relative, i.e. fp32-level accuracy.
//
// One CTA computes one 128 x BN output tile (optionally one K-split of it):
//   * 8 producer warps gather the operand tiles straight from global memory through a
//     loader functor (plain matrices in either orientation, or the implicit-GEMM views of
//     a convolution: no im2col buffer exists), split them into hi / lo and store both into
//     shared memory in the K-major, non-swizzled UMMA core-matrix layout (8 rows x 16 bytes
//     per core matrix; the stride between 8-row groups is padded by 16 bytes so that the
//     128-bit stores of both the K-contiguous and the transposing path are conflict free);
//   * one thread of a ninth warp issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8), three per
//     K-step, and signals stage reuse / accumulator completion with tcgen05.commit;
//   * the producer warps then read the accumulator with tcgen05.ld and write the result.
// Stages are handed over with mbarriers.  Every wait is bounded: on expiry the kernel
// records an error code in the context's status word, skips the rest of its work, still
// frees its TMEM columns and returns.
#include "rt_internal.cuh"
#include "conv_geom.cuh"
#include "tc_common.cuh"
#include <type_traits>

rt_status rt_sum_axis_internal(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out,
                               float scale);

namespace tc {

constexpr int BM = 128;          // UMMA M
constexpr int BK = 32;           // fp32 elements per stage along K (4 UMMA K-steps of 8)
constexpr int kProducerWarps = 8;
constexpr int kThreads = (kProducerWarps + 1) * 32;
constexpr uint32_t LBO = 128;    // bytes between core matrices along K
constexpr uint32_t SBO = (BK / 4) * 128 + 16;  // bytes between 8-row groups (padded: SBO/16 is odd)

__host__ __device__ constexpr uint32_t tile_bytes(int rows) { return (uint32_t)(rows / 8) * SBO; }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) { return make_desc(saddr, LBO, SBO); }

// ---- operand loaders -----------------------------------------------------------------------
// Rows are the M (A operand) or N (B operand) index.  A producer thread works on the same rows
// for the whole K loop, so everything that depends only on the row is decoded once into a small
// State (prep_*); the per-K-block fetch then costs a handful of integer instructions per load.
//   kKind 0 (K-contiguous):   State prep_row(row);        fetch_k4(state, k0, kend, v): 4 consecutive k
//   kKind 1 (row-contiguous): State prep_quad(first_row); fetch_r4(state, k, kend, v):  4 consecutive rows
//   kKind 2 (pixel rows):     State prep_quad(first_row); fetch_c4(state, q, qend, v):  for 4 consecutive rows the
//                             4 consecutive k of chunk q (k = 4q .. 4q+3)
// Out-of-range elements read as 0.
struct MatK {  // element(row, k) = p[row * ld + k]
  static constexpr int kKind = 0;
  const float* p;
  int64_t ld;
  int rows;
  bool vec;  // base and ld allow 16-byte loads
  struct State { const float* q; };
  __device__ __forceinline__ State prep_row(int row) const { return State{row < rows ? p + (int64_t)row * ld : nullptr}; }
  __device__ __forceinline__ void fetch_k4(const State& s, int k0, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (!s.q || k0 >= kend) return;
    if (vec && k0 + 3 < kend) {
      float4 t = __ldg(reinterpret_cast<const float4*>(s.q + k0));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (k0 + i < kend) v[i] = __ldg(s.q + k0 + i);
    }
  }
};
struct MatMN {  // element(row, k) = p[k * ld + row]
  static constexpr int kKind = 1;
  const float* p;
  int64_t ld;
  int rows;
  bool vec;
  struct State { int r0; };
  __device__ __forceinline__ State prep_quad(int r0) const { return State{r0}; }
  __device__ __forceinline__ void fetch_r4(const State& s, int k, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (k >= kend || s.r0 >= rows) return;
    const float* q = p + (int64_t)k * ld + s.r0;
    if (vec && s.r0 + 3 < rows) {
      float4 t = __ldg(reinterpret_cast<const float4*>(q));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (s.r0 + i < rows) v[i] = __ldg(q + i);
    }
  }
};

// ---- implicit-GEMM views of a convolution -----------------------------------------------------
// Geometry (conv_geom.cuh): wide tensor X[Nb,Cx,Hx,Wx], narrow tensor Y[Nb,Cy,Hy,Wy],
// y(b,cy,yo,xo) touches x(b,cx,yo*sh-ph+ky,xo*sw-pw+kx).  All element offsets fit in 31 bits
// (checked by the host dispatchers).

// Rows = output pixels (b,yo,xo), k = (cx,ky,kx): the im2col matrix of X, pixel-contiguous.
struct Im2colRows {
  static constexpr int kKind = 1;
  const float* x;
  ConvGeom g;
  int rows;
  struct State {
    int base[4];   // offset of x(b, 0, yo*sh-ph, xo*sw-pw) (may point outside the image)
    int iy0[4], ix0[4];
    int n;         // number of valid rows in the quad
  };
  __device__ __forceinline__ State prep_quad(int r0) const {
    State s;
    s.n = rows - r0 < 0 ? 0 : (rows - r0 > 4 ? 4 : rows - r0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b = 0, p = 0, yo = 0, xo = 0;
      if (i < s.n) {
        g.d_HyWy.divmod(r0 + i, b, p);
        g.d_Wy.divmod(p, yo, xo);
      }
      s.iy0[i] = (int)(yo * g.sh) - g.ph;
      s.ix0[i] = (int)(xo * g.sw) - g.pw;
      s.base[i] = ((int)b * g.Cx * g.Hx + s.iy0[i]) * g.Wx + s.ix0[i];
    }
    return s;
  }
  __device__ __forceinline__ void fetch_r4(const State& s, int k, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (k >= kend) return;
    uint32_t cx, r, ky, kx;
    g.d_khw.divmod(k, cx, r);
    g.d_kw.divmod(r, ky, kx);
    const int koff = ((int)cx * g.Hx + (int)ky) * g.Wx + (int)kx;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int iy = s.iy0[i] + (int)ky, ix = s.ix0[i] + (int)kx;
      if (i < s.n && iy >= 0 && iy < g.Hx && ix >= 0 && ix < g.Wx) v[i] = __ldg(x + s.base[i] + koff);
    }
  }
};

// Rows = input pixels (b,iy,ix), k = (cy,ky,kx): the gather of Y used by the input gradient and
// by the transposed convolution; element = y(b,cy,(iy+ph-ky)/sh,(ix+pw-kx)/sw) when exact and in range.
struct GatherRows {
  static constexpr int kKind = 1;
  const float* y;
  ConvGeom g;
  int rows;
  struct State {
    int base[4];  // offset of y(b, 0, 0, 0)
    int ty0[4], tx0[4];  // iy + ph, ix + pw
    int n;
  };
  __device__ __forceinline__ State prep_quad(int r0) const {
    State s;
    s.n = rows - r0 < 0 ? 0 : (rows - r0 > 4 ? 4 : rows - r0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b = 0, p = 0, iy = 0, ix = 0;
      if (i < s.n) {
        g.d_HxWx.divmod(r0 + i, b, p);
        g.d_Wx.divmod(p, iy, ix);
      }
      s.ty0[i] = (int)iy + g.ph;
      s.tx0[i] = (int)ix + g.pw;
      s.base[i] = (int)b * g.Cy * g.Hy * g.Wy;
    }
    return s;
  }
  __device__ __forceinline__ void fetch_r4(const State& s, int k, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (k >= kend) return;
    uint32_t cy, r, ky, kx;
    g.d_khw.divmod(k, cy, r);
    g.d_kw.divmod(r, ky, kx);
    const int coff = (int)cy * g.Hy * g.Wy;
    const bool unit = g.sh == 1 && g.sw == 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int ty = s.ty0[i] - (int)ky, tx = s.tx0[i] - (int)kx;
      if (i >= s.n || ty < 0 || tx < 0) continue;
      int yo = ty, xo = tx;
      if (!unit) {
        uint32_t q, rem;
        g.d_sh.divmod((uint32_t)ty, q, rem);
        if (rem) continue;
        yo = (int)q;
        g.d_sw.divmod((uint32_t)tx, q, rem);
        if (rem) continue;
        xo = (int)q;
      }
      if (yo < g.Hy && xo < g.Wy) v[i] = __ldg(y + s.base[i] + coff + yo * g.Wy + xo);
    }
  }
};

// Rows = cm, k = (cy, tap): weights stored [Cy, Cm, kh, kw] read with the second index as the row.
struct WeightSecondRows {
  static constexpr int kKind = 0;
  const float* w;
  ConvGeom g;
  int rows;  // Cm
  struct State { int off; };  // row * kh*kw, or -1
  __device__ __forceinline__ State prep_row(int row) const { return State{row < rows ? row * g.kh * g.kw : -1}; }
  __device__ __forceinline__ void fetch_k4(const State& s, int k0, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (s.off < 0 || k0 >= kend) return;
    const int khw = g.kh * g.kw;
    uint32_t cy, r;
    g.d_khw.divmod(k0, cy, r);
    int o = (int)cy * rows * khw + s.off + (int)r, rr = (int)r;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (k0 + i < kend) v[i] = __ldg(w + o);
      ++o;
      if (++rr == khw) {  // next channel of the narrow tensor
        rr = 0;
        o += (rows - 1) * khw;
      }
    }
  }
};

// Rows = (cx,ky,kx), k = output pixels (b,yo,xo): the im2col matrix with the pixel index as the
// reduction (weight gradient).  A thread walks eight consecutive pixels of its row with running
// coordinates, so the pixel index is decoded once per eight elements.
struct Im2colK4 {
  static constexpr int kKind = 0;
  static constexpr int kInvalid = -(1 << 30);
  const float* x;
  ConvGeom g;
  int rows;      // Cx*kh*kw
  int row_jump;  // offset change from the end of one output row to the start of the next: sh*Wx - Wy*sw
  int img_jump;  // from the end of one image to the start of the next: (Cx*Hx - Hy*sh)*Wx
  struct State { int coff, dy, dx; };  // dy = ky-ph, dx = kx-pw, coff = (cx*Hx + dy)*Wx + dx
  __device__ __forceinline__ State prep_row(int row) const {
    if (row >= rows) return State{0, kInvalid, 0};
    uint32_t cx, r, ky, kx;
    g.d_khw.divmod(row, cx, r);
    g.d_kw.divmod(r, ky, kx);
    const int dy = (int)ky - g.ph, dx = (int)kx - g.pw;
    return State{((int)cx * g.Hx + dy) * g.Wx + dx, dy, dx};
  }
  __device__ __forceinline__ void fetch_k8(const State& s, int k0, int kend, float (&v0)[4], float (&v1)[4]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) v0[i] = v1[i] = 0.f;
    if (s.dy == kInvalid || k0 >= kend) return;
    const int n = kend - k0;
    uint32_t b, p, yo, xo;
    g.d_HyWy.divmod(k0, b, p);
    g.d_Wy.divmod(p, yo, xo);
    int iy = (int)yo * g.sh + s.dy, ix = (int)xo * g.sw + s.dx;
    int off = ((int)b * g.Cx * g.Hx + (int)yo * g.sh) * g.Wx + (int)xo * g.sw + s.coff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float t = 0.f;
      if (i < n && (unsigned)iy < (unsigned)g.Hx && (unsigned)ix < (unsigned)g.Wx) t = __ldg(x + off);
      if (i < 4) v0[i] = t; else v1[i - 4] = t;
      ix += g.sw;
      off += g.sw;
      if ((int)++xo == g.Wy) {  // next output row / next image
        xo = 0;
        ix = s.dx;
        off += row_jump;
        iy += g.sh;
        if ((int)++yo == g.Hy) {
          yo = 0;
          iy = s.dy;
          off += img_jump;
        }
      }
    }
  }
};

// Rows = cy, k = pixels (b,p): the narrow tensor with the pixel index as the reduction.
struct NarrowK4 {
  static constexpr int kKind = 0;
  const float* y;
  ConvGeom g;
  int rows;  // Cy
  bool vec;  // Hy*Wy % 4 == 0 and y is 16-byte aligned
  struct State { int off; };  // row * Hy*Wy or -1
  __device__ __forceinline__ State prep_row(int row) const { return State{row < rows ? row * g.Hy * g.Wy : -1}; }
  __device__ __forceinline__ void fetch_k4(const State& s, int k0, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (s.off < 0 || k0 >= kend) return;
    const int hw = g.Hy * g.Wy;
    uint32_t b, p;
    g.d_HyWy.divmod(k0, b, p);
    if (vec && k0 + 3 < kend) {  // k0 % 4 == 0 and hw % 4 == 0: the four pixels share one image
      float4 t = __ldg(reinterpret_cast<const float4*>(y + (int)b * g.Cy * hw + s.off + (int)p));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + i < kend) v[i] = __ldg(y + (int)b * g.Cy * hw + s.off + (int)p);
        if ((int)++p == hw) {
          p = 0;
          ++b;
        }
      }
    }
  }
};

// Rows = pixels (b,yo,xo) of the narrow side of a convolution-shaped gather from src[Nb,C,H,W]:
// the row reads src(b, c, yo*sh-ph+ky, xo*sw-pw+kx).  The reduction index is laid out as
// k = ((c*kh + ky)*kwq + kxq)*4 + j with the kernel columns padded to kwq*4 >= kw, so that one
// 16-byte K-chunk of a row is four consecutive source columns of one source row: a chunk costs one
// row test, one address and four predicated loads; the column tests are a per-pixel bit mask
// computed once.  The padding columns are zeros in both operands.
struct PixelTapRows {
  static constexpr int kKind = 2;
  const float* src;
  int C, H, W;           // source channels / height / width
  int kh, kw, kwq;       // kernel extent, number of 4-wide column chunks
  int sh, sw, ph, pw;
  int rows;              // Nb * rows_h * rows_w
  FastDiv d_hw, d_w;     // pixels per image / per row on the row side
  FastDiv d_kh, d_kwq;
  struct State {
    int base[4];         // offset of src(b, 0, yo*sh-ph, xo*sw-pw) (may lie outside the image)
    int iy0[4];
    uint32_t cmask[4];   // bit t: kernel column t exists and falls inside the source row
  };
  __device__ __forceinline__ State prep_quad(int r0) const {
    State s;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s.base[i] = 0;
      s.iy0[i] = 0;
      s.cmask[i] = 0;
      if (r0 + i < rows) {
        uint32_t b, p, yo, xo;
        d_hw.divmod(r0 + i, b, p);
        d_w.divmod(p, yo, xo);
        const int iy0 = (int)yo * sh - ph, ix0 = (int)xo * sw - pw;
        s.iy0[i] = iy0;
        s.base[i] = ((int)b * C * H + iy0) * W + ix0;
        uint32_t m = 0;
        for (int t = 0; t < kw; ++t)
          if ((unsigned)(ix0 + t) < (unsigned)W) m |= 1u << t;
        s.cmask[i] = m;
      }
    }
    return s;
  }
  __device__ __forceinline__ void fetch_c4(const State& s, int q, int qend, float (&v)[4][4]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) v[i][j] = 0.f;
    if (q >= qend) return;
    uint32_t ck, kxq, c, ky;
    d_kwq.divmod(q, ck, kxq);
    d_kh.divmod(ck, c, ky);
    const int koff = ((int)c * H + (int)ky) * W + (int)kxq * 4;
    const int shift = (int)kxq * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int iy = s.iy0[i] + (int)ky;
      const uint32_t m = (unsigned)iy < (unsigned)H ? (s.cmask[i] >> shift) & 15u : 0u;
      const float* p = src + s.base[i] + koff;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (m & (1u << j)) v[i][j] = __ldg(p + j);
    }
  }
};

// Weights in the padded tap order of PixelTapRows: element(row n, k = ((c*kh+ky)*kwq+kxq)*4+j) =
// w[n*sn + c*sc + ky*sky + kx*skx + off0] for kx = kxq*4+j < kw, else 0.  Strides may be negative
// (flipped kernels of the input gradient).
struct TapWeights {
  static constexpr int kKind = 0;
  const float* w;
  int rows, kh, kw, kwq;
  int sn, sc, sky, skx, off0;
  FastDiv d_kh, d_kwq;
  struct State { int off; };  // n*sn + off0, or -1
  __device__ __forceinline__ State prep_row(int row) const { return State{row < rows ? row * sn + off0 : -1}; }
  __device__ __forceinline__ void fetch_k4(const State& s, int k0, int kend, float (&v)[4]) const {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (s.off < 0 || k0 >= kend) return;
    uint32_t ck, kxq, c, ky;
    d_kwq.divmod(k0 >> 2, ck, kxq);
    d_kh.divmod(ck, c, ky);
    const float* p = w + s.off + (int)c * sc + (int)ky * sky;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kx = (int)kxq * 4 + j;
      if (kx < kw) v[j] = __ldg(p + kx * skx);
    }
  }
};

// ---- epilogues -------------------------------------------------------------------------------
struct PlainOut {  // c[z * split_stride + m * ld + n]
  float* c;
  int64_t ld, split_stride;
  int M, N;
  bool accumulate;
  __device__ __forceinline__ void store32(int m, int n0, const float (&v)[32], int z) const {
    if (m >= M) return;
    float* q = c + z * split_stride + (int64_t)m * ld + n0;
    bool vec4 = (n0 + 31 < N) && ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
    if (vec4 && !accumulate) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(q + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else if (vec4) {  // accumulate: all eight 128-bit loads of the old values are issued before the first add
      float4 old[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) old[j] = *reinterpret_cast<const float4*>(q + 4 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(q + 4 * j) =
            make_float4(old[j].x + v[4 * j], old[j].y + v[4 * j + 1], old[j].z + v[4 * j + 2], old[j].w + v[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + j < N) q[j] = accumulate ? q[j] + v[j] : v[j];
    }
  }
};
struct ImageOut {  // out[b, n, p] for row m = (b,p), optional per-channel bias
  float* out;
  const float* bias;
  int C, HW, M;
  FastDiv d_HW;
  __device__ __forceinline__ void store32(int m, int n0, const float (&v)[32], int) const {
    if (m >= M) return;
    uint32_t b, p;
    d_HW.divmod(m, b, p);
    float* q = out + ((int64_t)b * C + n0) * HW + p;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n0 + j < C) q[(int64_t)j * HW] = bias ? v[j] + __ldg(bias + n0 + j) : v[j];
  }
};
struct PhaseOut {  // out[b, n, j*sy + oy, i*sx + ox] for row m = (b, j, i) of one stride phase, optional per-channel bias
  float* out;
  const float* bias;
  int C, Hfull, Wfull, sy, sx, oy, ox, M;
  FastDiv d_HjWj, d_Wj;
  __device__ __forceinline__ void store32(int m, int n0, const float (&v)[32], int) const {
    if (m >= M) return;
    uint32_t b, r, j, i;
    d_HjWj.divmod(m, b, r);
    d_Wj.divmod(r, j, i);
    const int64_t hw = (int64_t)Hfull * Wfull;
    float* q = out + ((int64_t)b * C + n0) * hw + (int64_t)((int)j * sy + oy) * Wfull + (int)i * sx + ox;
#pragma unroll
    for (int jn = 0; jn < 32; ++jn)
      if (n0 + jn < C) q[(int64_t)jn * hw] = bias ? v[jn] + __ldg(bias + n0 + jn) : v[jn];
  }
};
struct TransposedOut {  // c[z * split_stride + n * ld + m]: the tile is written transposed
  float* c;
  int64_t ld, split_stride;
  int M, N;
  __device__ __forceinline__ void store32(int m, int n0, const float (&v)[32], int z) const {
    if (m >= M) return;
    float* q = c + z * split_stride + (int64_t)n0 * ld + m;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n0 + j < N) q[(int64_t)j * ld] = v[j];
  }
};

// ---- per-thread producer of one operand tile (ROWS x BK) --------------------------------------
// fetch() reads this thread's share of a K-block from global memory into registers; commit()
// splits it into hi / lo and stores both in the UMMA layout.  The kernel keeps two register
// buffers so that the loads of K-block i+1 are in flight while K-block i is converted.
template <class L, class = void>
struct HasFetchK8 : std::false_type {};
template <class L>
struct HasFetchK8<L, std::void_t<decltype(&L::fetch_k8)>> : std::true_type {};
template <class L>
__device__ __forceinline__ void fetch_k8(const L& ld, const typename L::State& s, int k0, int kend, float (&v0)[4],
                                         float (&v1)[4]) {
  if constexpr (HasFetchK8<L>::value) {
    ld.fetch_k8(s, k0, kend, v0, v1);
  } else {
    ld.fetch_k4(s, k0, kend, v0);
    ld.fetch_k4(s, k0 + 4, kend, v1);
  }
}

template <int ROWS, class L, int KIND = L::kKind>
struct Producer;

// K-contiguous source: item = (row group of 8, row in group, group of 8 k).  Lanes run along rows
// so that each quarter-warp writes one whole 128-byte core matrix (conflict free); a lane reads 32 B.
template <int ROWS, class L>
struct Producer<ROWS, L, 0> {
  static constexpr int kItems = (ROWS / 8 + kProducerWarps - 1) / kProducerWarps;
  typename L::State st[kItems];
  int warp, r8, kg;
  struct Buf { float v[kItems][2][4]; };
  __device__ __forceinline__ void init(const L& ld, int row0, int w, int lane) {
    warp = w; r8 = lane & 7; kg = lane >> 3;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int rg = warp + j * kProducerWarps;
      st[j] = ld.prep_row(rg < ROWS / 8 ? row0 + rg * 8 + r8 : 0x7fffffff);
    }
  }
  __device__ __forceinline__ void fetch(const L& ld, int k0, int kend, Buf& b) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j)
      if (warp + j * kProducerWarps < ROWS / 8) {
        fetch_k8(ld, st[j], k0 + kg * 8, kend, b.v[j][0], b.v[j][1]);
      }
  }
  __device__ __forceinline__ void commit(const Buf& b, char* hi, char* lo) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int rg = warp + j * kProducerWarps;
      if (rg < ROWS / 8) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float4 vh, vl;
          split4(b.v[j][h], vh, vl);
          const uint32_t off = (uint32_t)rg * SBO + (uint32_t)(kg * 2 + h) * LBO + (uint32_t)r8 * 16;
          *reinterpret_cast<float4*>(hi + off) = vh;
          *reinterpret_cast<float4*>(lo + off) = vl;
        }
      }
    }
  }
};

// Row-contiguous source: item = (quad of rows, quad of k): a 4x4 block is fetched as four
// row-vectors, transposed in registers and written as four 16-byte K-vectors.
template <int ROWS, class L>
struct Producer<ROWS, L, 1> {
  static constexpr int kTotal = (ROWS / 4) * (BK / 4);
  static constexpr int kItems = (kTotal + kProducerWarps * 32 - 1) / (kProducerWarps * 32);
  typename L::State st[kItems];
  int tid;
  struct Buf { float v[kItems][4][4]; };
  __device__ __forceinline__ void init(const L& ld, int row0, int w, int lane) {
    tid = w * 32 + lane;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      st[j] = ld.prep_quad(item < kTotal ? row0 + (item % (ROWS / 4)) * 4 : 0x7ffffff0);
    }
  }
  __device__ __forceinline__ void fetch(const L& ld, int k0, int kend, Buf& b) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      if (item < kTotal) {
        int kq = item / (ROWS / 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) ld.fetch_r4(st[j], k0 + kq * 4 + i, kend, b.v[j][i]);
      }
    }
  }
  __device__ __forceinline__ void commit(const Buf& b, char* hi, char* lo) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      if (item < kTotal) {
        int rq = item % (ROWS / 4), kq = item / (ROWS / 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v[4] = {b.v[j][0][i], b.v[j][1][i], b.v[j][2][i], b.v[j][3][i]};
          float4 vh, vl;
          split4(v, vh, vl);
          const int row = rq * 4 + i;
          const uint32_t off = (uint32_t)(row >> 3) * SBO + (uint32_t)kq * LBO + (uint32_t)(row & 7) * 16;
          *reinterpret_cast<float4*>(hi + off) = vh;
          *reinterpret_cast<float4*>(lo + off) = vl;
        }
      }
    }
  }
};

// Pixel-row source with K-chunks: item = (quad of rows, chunk of 4 k).  The loader already returns
// each row's four consecutive k, so the registers go to shared memory without a transpose.
template <int ROWS, class L>
struct Producer<ROWS, L, 2> {
  static constexpr int kTotal = (ROWS / 4) * (BK / 4);
  static constexpr int kItems = (kTotal + kProducerWarps * 32 - 1) / (kProducerWarps * 32);
  typename L::State st[kItems];
  int tid;
  struct Buf { float v[kItems][4][4]; };
  __device__ __forceinline__ void init(const L& ld, int row0, int w, int lane) {
    tid = w * 32 + lane;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      st[j] = ld.prep_quad(item < kTotal ? row0 + (item % (ROWS / 4)) * 4 : 0x7ffffff0);
    }
  }
  __device__ __forceinline__ void fetch(const L& ld, int k0, int kend, Buf& b) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      if (item < kTotal) ld.fetch_c4(st[j], (k0 >> 2) + item / (ROWS / 4), (kend + 3) >> 2, b.v[j]);
    }
  }
  __device__ __forceinline__ void commit(const Buf& b, char* hi, char* lo) const {
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      int item = tid + j * kProducerWarps * 32;
      if (item < kTotal) {
        int rq = item % (ROWS / 4), kq = item / (ROWS / 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float4 vh, vl;
          split4(b.v[j][i], vh, vl);
          const int row = rq * 4 + i;
          const uint32_t off = (uint32_t)(row >> 3) * SBO + (uint32_t)kq * LBO + (uint32_t)(row & 7) * 16;
          *reinterpret_cast<float4*>(hi + off) = vh;
          *reinterpret_cast<float4*>(lo + off) = vl;
        }
      }
    }
  }
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr uint32_t a_bytes = tile_bytes(BM), b_bytes = tile_bytes(BN);
  static constexpr uint32_t stage_bytes = 2 * a_bytes + 2 * b_bytes;  // A hi, A lo, B hi, B lo
  static constexpr uint32_t bar_offset = STAGES * stage_bytes;
  static constexpr uint32_t total = bar_offset + (2 * STAGES + 1) * 8 + 16;
};

template <int BN, int STAGES, class LA, class LB, class EPI>
__global__ void __launch_bounds__(kThreads, (BN <= 64 && STAGES <= 2) ? 2 : 1)
tc_gemm_kernel(const LA la, const LB lb, const EPI epi, int K, int k_per_split, int* status) {
  extern __shared__ __align__(128) char smem[];
  using SL = SmemLayout<BN, STAGES>;
  // Four accumulators per tile, BN columns each.  The tensor core adds every K=8 partial product
  // into the fp32 accumulator with truncation, an error that grows linearly with the number of
  // additions and with the accumulator's magnitude; spreading the hi*hi products round-robin over
  // three accumulators and keeping the small cross terms (hi*lo, lo*hi) in a fourth one cuts that
  // error several times.  The epilogue adds the four in round-to-nearest fp32.
  constexpr int kAccs = 4;
  constexpr uint32_t kTmemCols = kAccs * BN;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM allocation must be a power of two <= 512");
  // broadcast from lane 0 so that the compiler knows the value is the same in every lane (uniform role branches and registers)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kbeg = blockIdx.z * k_per_split;
  const int kend = min(K, kbeg + k_per_split);
  const int nkb = (kend - kbeg + BK - 1) / BK;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bars = smem_base + SL::bar_offset;  // full[s], empty[s], acc
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SL::bar_offset + (2 * STAGES + 1) * 8);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bars + 8 * s, kProducerWarps);
      mbar_init(bars + 8 * (STAGES + s), 1);
    }
    mbar_init(bars + 8 * (2 * STAGES), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kProducerWarps) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  bool ok = true;
  if (warp < kProducerWarps) {
    // ---------------- producers ----------------
    Producer<BM, LA> pa;
    Producer<BN, LB> pb;
    pa.init(la, m0, warp, lane);
    pb.init(lb, n0, warp, lane);
    typename Producer<BM, LA>::Buf a0, a1;
    typename Producer<BN, LB>::Buf b0, b1;
    auto stage_out = [&](int it, const typename Producer<BM, LA>::Buf& ba, const typename Producer<BN, LB>::Buf& bb) -> bool {
      const int s = it % STAGES;
      if (it >= STAGES && !mbar_wait(bars + 8 * (STAGES + s), ((it / STAGES) - 1) & 1, status, 1)) return false;
      char* st = smem + s * SL::stage_bytes;
      pa.commit(ba, st, st + SL::a_bytes);
      pb.commit(bb, st + 2 * SL::a_bytes, st + 2 * SL::a_bytes + SL::b_bytes);
      fence_async_smem();  // make the generic-proxy stores visible to the tensor-core (async) proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * s);
      return true;
    };
    if (nkb > 0) {
      pa.fetch(la, kbeg, kend, a0);
      pb.fetch(lb, kbeg, kend, b0);
    }
    for (int it = 0; it < nkb && ok; it += 2) {
      if (it + 1 < nkb) {
        pa.fetch(la, kbeg + (it + 1) * BK, kend, a1);
        pb.fetch(lb, kbeg + (it + 1) * BK, kend, b1);
      }
      ok = stage_out(it, a0, b0);
      if (ok && it + 1 < nkb) {
        if (it + 2 < nkb) {
          pa.fetch(la, kbeg + (it + 2) * BK, kend, a0);
          pb.fetch(lb, kbeg + (it + 2) * BK, kend, b0);
        }
        ok = stage_out(it + 1, a1, b1);
      }
    }
    // ---------------- epilogue ----------------
    if (ok && nkb > 0) ok = mbar_wait(bars + 8 * (2 * STAGES), 0, status, 2);
    tc_fence_after();
    if (ok) {
      const int quad = warp & 3, half = warp >> 2;
      constexpr int chunks = BN / 32 > 0 ? BN / 32 : 1;
      const int m = m0 + quad * 32 + lane;
      for (int c = half; c < chunks; c += 2) {
        float v[32];
        if (nkb > 0) {
          const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
          tmem_ld32(t0, v);  // cross terms
#pragma unroll
          for (int a = 1; a < kAccs; ++a) {
            float u[32];
            tmem_ld32(t0 + (uint32_t)(a * BN), u);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += u[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        epi.store32(m, n0 + c * 32, v, blockIdx.z);
      }
    }
  } else {
    // ---------------- MMA issuer: the whole warp runs the loop (operands stay warp-uniform), one elected lane issues ----
    constexpr uint32_t idesc = make_idesc(BN);
    const uint32_t hi32 = desc_hi32(SBO);
    uint32_t rot = 0;  // hi*hi accumulator 1 + rot
    for (int it = 0; it < nkb && ok; ++it) {
      const int s = it % STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * s, (it / STAGES) & 1, status, 3));
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_hi = desc_lo32(smem_base + s * SL::stage_bytes, LBO), a_lo = a_hi + (SL::a_bytes >> 4);
      const uint32_t b_hi = a_hi + ((2 * SL::a_bytes) >> 4), b_lo = b_hi + (SL::b_bytes >> 4);
#pragma unroll
      for (int j = 0; j < BK / 8; ++j) {
        const uint32_t ko = (uint32_t)j * ((2 * LBO) >> 4);
        const int t = it * (BK / 8) + j;  // K-step counter of this tile
        // cross terms -> accumulator 0, hi*hi round-robin -> accumulators 1..3
        umma_tf32_step_elect(tmem_base, tmem_base + (1 + rot) * BN, a_hi + ko, a_lo + ko, hi32, b_hi + ko, b_lo + ko, hi32, idesc,
                             t != 0 ? 1u : 0u, t >= 3 ? 1u : 0u);
        rot = rot == 2 ? 0 : rot + 1;
      }
      umma_commit_elect(bars + 8 * (STAGES + s));  // frees the stage when these MMAs have read it
    }
    if (ok && nkb > 0) umma_commit_elect(bars + 8 * (2 * STAGES));  // accumulator complete
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- plain products with the A operand in tensor memory (TS form) -----------------------------------------------------
// tc_gemm_kernel stages the hi / lo images of BOTH operands in shared memory and is bound by its bandwidth: per K-block of 32 the
// producers write 64 KB and the twelve MMAs read 96 KB through a 128 B/cycle path (1 250 cycles against 780 cycles of tensor
// work; measured 2 350 cycles per K-block).  Here the A tile never touches shared memory: every producer thread owns one row of
// the tile (= one lane of tensor memory), loads 16 of its 32 k-values, splits them and writes hi and lo straight into tensor
// memory with tcgen05.st; the MMAs read A from there (an MMA with A in tensor memory costs N/2 cycles for every N) and only
// the 64-column B tile crosses shared memory (16 KB written, 24 KB read per K-block).  Used for products whose grid is small
// enough to be latency-bound (the fully connected and recurrent layers); large products keep the 128 x 128 tile, whose wider B
// tile halves the traffic from L2.
struct PlainA {  // element(row, k) = trans ? p[k * ld + row] : p[row * ld + k]
  const float* p;
  int64_t ld;
  int rows;
  bool trans, vec;
};
constexpr int kTsBN = 64, kTsStages = 3, kTsAccs = 4;
constexpr uint32_t kTsAccCols = kTsAccs * kTsBN;        // 256 accumulator columns
constexpr uint32_t kTsAStageCols = 2 * BK;              // hi k 0..31, lo k 0..31
struct TsSmem {
  static constexpr uint32_t b_bytes = tile_bytes(kTsBN);
  static constexpr uint32_t stage_bytes = 2 * b_bytes;  // B hi, B lo
  static constexpr uint32_t bar_offset = kTsStages * stage_bytes;
  static constexpr uint32_t total = bar_offset + (2 * kTsStages + 1) * 8 + 16;
};
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
      "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// One 3xTF32 K-step with A in tensor memory: lo*hi and hi*lo into the cross accumulator, hi*hi into the main one.
__device__ __forceinline__ void umma_tf32_step_ts_elect(uint32_t d_cross, uint32_t d_main, uint32_t a_hi_t, uint32_t a_lo_t, uint32_t b_hi_lo32,
                                                        uint32_t b_lo_lo32, uint32_t b_hi32, uint32_t idesc, uint32_t acc_cross,
                                                        uint32_t acc_main) {
  asm volatile(
      "{\n\t.reg .pred pc, pm, pt, pe;\n\t"
      ".reg .b64 dbh, dbl;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pc, %8, 0;\n\t"
      "setp.ne.b32 pm, %9, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 dbh, {%4, %6};\n\t"
      "mov.b64 dbl, {%5, %6};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%3], dbh, %7, pc;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], dbl, %7, pt;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%1], [%2], dbh, %7, pm;\n\t}" ::"r"(d_cross), "r"(d_main), "r"(a_hi_t), "r"(a_lo_t),
      "r"(b_hi_lo32), "r"(b_lo_lo32), "r"(b_hi32), "r"(idesc), "r"(acc_cross), "r"(acc_main)
      : "memory");
}

template <class LB, class EPI>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_ts_kernel(const PlainA la, const LB lb, const EPI epi, int K, int k_per_split, int* status) {
  extern __shared__ __align__(128) char smem[];
  using SL = TsSmem;
  constexpr int BN = kTsBN, STAGES = kTsStages;
  // broadcast from lane 0 so that the compiler knows the value is the same in every lane (uniform role branches and registers)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kbeg = blockIdx.z * k_per_split;
  const int kend = min(K, kbeg + k_per_split);
  const int nkb = (kend - kbeg + BK - 1) / BK;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bars = smem_base + SL::bar_offset;  // full[s], empty[s], acc
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SL::bar_offset + (2 * STAGES + 1) * 8);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bars + 8 * s, kProducerWarps);
      mbar_init(bars + 8 * (STAGES + s), 1);
    }
    mbar_init(bars + 8 * (2 * STAGES), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kProducerWarps) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  const uint32_t tmem_a = tmem_base + kTsAccCols;  // A stages behind the accumulators

  bool ok = true;
  if (warp < kProducerWarps) {
    // ---------------- producers: every thread one row of A (16 k-values) and its share of the B tile ----------------
    const int quad = warp & 3, khalf = warp >> 2;
    const int row = m0 + quad * 32 + lane;
    const bool row_ok = row < la.rows;
    const float* arow = la.trans ? la.p + row : la.p + (int64_t)row * la.ld;
    Producer<BN, LB> pb;
    pb.init(lb, n0, warp, lane);
    struct ABuf { float v[16]; };
    auto fetch_a = [&](int k0, ABuf& b) {
      const int kk = k0 + khalf * 16;
#pragma unroll
      for (int i = 0; i < 16; ++i) b.v[i] = 0.f;
      if (!row_ok || kk >= kend) return;
      if (!la.trans) {
        if (la.vec && kk + 15 < kend) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(arow + kk) + j);
            b.v[4 * j] = t.x; b.v[4 * j + 1] = t.y; b.v[4 * j + 2] = t.z; b.v[4 * j + 3] = t.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (kk + i < kend) b.v[i] = __ldg(arow + kk + i);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (kk + i < kend) b.v[i] = __ldg(arow + (int64_t)(kk + i) * la.ld);  // consecutive lanes read consecutive rows
      }
    };
    ABuf a0, a1;
    typename Producer<BN, LB>::Buf b0, b1;
    auto stage_out = [&](int it, const ABuf& ba, const typename Producer<BN, LB>::Buf& bb) -> bool {
      const int s = it % STAGES;
      if (it >= STAGES && !mbar_wait(bars + 8 * (STAGES + s), ((it / STAGES) - 1) & 1, status, 1)) return false;
      char* st = smem + s * SL::stage_bytes;
      pb.commit(bb, st, st + SL::b_bytes);
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t h = __float_as_uint(ba.v[i]) & 0xFFFFE000u;
        hi[i] = h;
        lo[i] = __float_as_uint(ba.v[i] - __uint_as_float(h));
      }
      const uint32_t ta = tmem_a + ((uint32_t)(quad * 32) << 16) + (uint32_t)s * kTsAStageCols + (uint32_t)khalf * 16;
      tmem_st16(ta, hi);
      tmem_st16(ta + BK, lo);
      tmem_wait_st();
      fence_async_smem();  // the B stores -> async proxy
      tc_fence_before();   // the tensor-memory stores are ordered before the arrive
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * s);
      return true;
    };
    if (nkb > 0) {
      fetch_a(kbeg, a0);
      pb.fetch(lb, kbeg, kend, b0);
    }
    for (int it = 0; it < nkb && ok; it += 2) {
      if (it + 1 < nkb) {
        fetch_a(kbeg + (it + 1) * BK, a1);
        pb.fetch(lb, kbeg + (it + 1) * BK, kend, b1);
      }
      ok = stage_out(it, a0, b0);
      if (ok && it + 1 < nkb) {
        if (it + 2 < nkb) {
          fetch_a(kbeg + (it + 2) * BK, a0);
          pb.fetch(lb, kbeg + (it + 2) * BK, kend, b0);
        }
        ok = stage_out(it + 1, a1, b1);
      }
    }
    // ---------------- epilogue ----------------
    if (ok && nkb > 0) ok = mbar_wait(bars + 8 * (2 * STAGES), 0, status, 2);
    tc_fence_after();
    if (ok) {
      const int m = m0 + quad * 32 + lane;
      const int c = khalf;  // two chunks of 32 columns: warps 0-3 the first, warps 4-7 the second
      float v[32];
      if (nkb > 0) {
        const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
        tmem_ld32(t0, v);  // cross terms
#pragma unroll
        for (int a = 1; a < kTsAccs; ++a) {
          float u[32];
          tmem_ld32(t0 + (uint32_t)(a * BN), u);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += u[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      }
      epi.store32(m, n0 + c * 32, v, blockIdx.z);
    }
  } else {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc(BN);
    const uint32_t hi32 = desc_hi32(SBO);
    uint32_t rot = 0;
    for (int it = 0; it < nkb && ok; ++it) {
      const int s = it % STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * s, (it / STAGES) & 1, status, 3));
      if (!ok) break;
      tc_fence_after();
      const uint32_t b_hi = desc_lo32(smem_base + s * SL::stage_bytes, LBO), b_lo = b_hi + (SL::b_bytes >> 4);
      const uint32_t a_hi = tmem_a + (uint32_t)s * kTsAStageCols, a_lo = a_hi + BK;
#pragma unroll
      for (int j = 0; j < BK / 8; ++j) {
        const uint32_t ko = (uint32_t)j * ((2 * LBO) >> 4);
        const int t = it * (BK / 8) + j;
        umma_tf32_step_ts_elect(tmem_base, tmem_base + (1 + rot) * BN, a_hi + 8 * j, a_lo + 8 * j, b_hi + ko, b_lo + ko, hi32, idesc,
                                t != 0 ? 1u : 0u, t >= 3 ? 1u : 0u);
        rot = rot == 2 ? 0 : rot + 1;
      }
      umma_commit_elect(bars + 8 * (STAGES + s));  // frees the B stage and the A slot when these MMAs have read them
    }
    if (ok && nkb > 0) umma_commit_elect(bars + 8 * (2 * STAGES));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <class LB, class EPI>
rt_status launch_ts(rt_ctx* ctx, const PlainA& la, const LB& lb, const EPI& epi, int M, int N, int K, int splits, int kps) {
  auto kern = tc_gemm_ts_kernel<LB, EPI>;
  RT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TsSmem::total));
  dim3 grid((N + kTsBN - 1) / kTsBN, (M + BM - 1) / BM, splits);
  kern<<<grid, kThreads, TsSmem::total, ctx->stream>>>(la, lb, epi, K, kps, ctx->device_status);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

template <int BN, int STAGES, class LA, class LB, class EPI>
rt_status launch(rt_ctx* ctx, const LA& la, const LB& lb, const EPI& epi, int M, int N, int K, int splits, int kps) {
  using SL = SmemLayout<BN, STAGES>;
  auto kern = tc_gemm_kernel<BN, STAGES, LA, LB, EPI>;
  RT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SL::total));
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
  kern<<<grid, kThreads, SL::total, ctx->stream>>>(la, lb, epi, K, kps, ctx->device_status);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

template <class LA, class LB, class EPI>
rt_status dispatch_bn(rt_ctx* ctx, const LA& la, const LB& lb, const EPI& epi, int M, int N, int K, int splits, int kps) {
  // Two shared-memory stages everywhere (the register double buffer hides the global latency);
  // tiles up to 64 columns then fit two CTAs per SM.
  if (N <= 32) return launch<32, 2>(ctx, la, lb, epi, M, N, K, splits, kps);
  if (N <= 64) return launch<64, 2>(ctx, la, lb, epi, M, N, K, splits, kps);
  return launch<128, 2>(ctx, la, lb, epi, M, N, K, splits, kps);
}

inline int n_tiles(int64_t M, int64_t N) {
  int bn = N <= 32 ? 32 : (N <= 64 ? 64 : 128);
  return (int)(((M + BM - 1) / BM) * ((N + bn - 1) / bn));
}

// Split-K policy: about two CTAs per SM in flight, at least 4 K-blocks per split.
inline void choose_split(rt_ctx* ctx, int64_t M, int64_t N, int64_t K, int* splits, int* kps) {
  int tiles = n_tiles(M, N);
  int64_t want = ((int64_t)ctx->sm_count * 2 + tiles - 1) / tiles;
  int64_t max_s = K / (4 * BK);
  if (max_s < 1) max_s = 1;
  int64_t s = want < max_s ? want : max_s;
  if (s < 1) s = 1;
  if (s > 512) s = 512;
  int64_t per = (K + s - 1) / s;
  per = (per + BK - 1) / BK * BK;
  s = (K + per - 1) / per;
  *splits = (int)(s < 1 ? 1 : s);
  *kps = (int)per;
}

// C[M,N] row-major = A x B with the given loaders; split-K through a workspace when useful.
template <class LA, class LB>
rt_status gemm_plain(rt_ctx* ctx, const LA& la, const LB& lb, float* c, int64_t ldc, int64_t M, int64_t N, int64_t K,
                     bool accumulate) {
  int splits = 1, kps = (int)((K + BK - 1) / BK * BK);
  if (!accumulate && ldc == N) choose_split(ctx, M, N, K, &splits, &kps);
  if (splits == 1) {
    PlainOut epi{c, ldc, 0, (int)M, (int)N, accumulate};
    return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, 1, kps);
  }
  RtScratch ws(ctx);
  rt_status st = ws.alloc(sizeof(float) * (size_t)splits * M * N);
  if (st != RT_OK) return st;
  PlainOut epi{ws.as<float>(), N, M * N, (int)M, (int)N, false};
  st = dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, splits, kps);
  if (st != RT_OK) return st;
  return rt_sum_axis_internal(ctx, ws.as<float>(), 1, splits, M * N, c, 1.f);
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The tensor-memory variant for products whose grid of 128 x 64 tiles fits one wave (one CTA per SM: the kernel takes all of
// tensor memory): they are bound by latency and by the staging of the operands, not by the traffic from L2.  Measured on the
// fully connected layer of the CNN (256 x 3136 x 128): 14.2 -> 11.2, 13.7 -> 9.4, 11.9 -> 10.2 us for forward, dX, dW; a K-block
// costs 0.16 us instead of 1.1.  RT_B200_GEMM_TS=0 turns it off, =2 uses it for every plain product.
inline bool use_ts_tile(rt_ctx* ctx, int64_t M, int64_t N) {
  static const int mode = [] {
    const char* e = getenv("RT_B200_GEMM_TS");
    return e && e[0] ? atoi(e) : 1;
  }();
  if (mode == 0) return false;
  if (mode >= 2) return true;
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + kTsBN - 1) / kTsBN);
  return tiles <= (int64_t)ctx->sm_count;
}
template <class LB>
rt_status gemm_plain_ts(rt_ctx* ctx, const PlainA& la, const LB& lb, float* c, int64_t ldc, int64_t M, int64_t N, int64_t K,
                        bool accumulate) {
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + kTsBN - 1) / kTsBN);
  int splits = 1, kps = (int)((K + BK - 1) / BK * BK);
  if (!accumulate && ldc == N) {  // one CTA per SM (the kernel takes all of tensor memory); at least 4 K-blocks per split
    int64_t want = ((int64_t)ctx->sm_count + tiles - 1) / tiles;
    int64_t max_s = K / (4 * BK);
    if (max_s < 1) max_s = 1;
    int64_t sp = want < max_s ? want : max_s;
    if (sp < 1) sp = 1;
    if (sp > 512) sp = 512;
    int64_t per = (K + sp - 1) / sp;
    per = (per + BK - 1) / BK * BK;
    sp = (K + per - 1) / per;
    splits = (int)(sp < 1 ? 1 : sp);
    kps = (int)per;
  }
  if (splits == 1) {
    PlainOut epi{c, ldc, 0, (int)M, (int)N, accumulate};
    return launch_ts(ctx, la, lb, epi, (int)M, (int)N, (int)K, 1, kps);
  }
  RtScratch ws(ctx);
  rt_status st = ws.alloc(sizeof(float) * (size_t)splits * M * N);
  if (st != RT_OK) return st;
  PlainOut epi{ws.as<float>(), N, M * N, (int)M, (int)N, false};
  st = launch_ts(ctx, la, lb, epi, (int)M, (int)N, (int)K, splits, kps);
  if (st != RT_OK) return st;
  return rt_sum_axis_internal(ctx, ws.as<float>(), 1, splits, M * N, c, 1.f);
}

inline PixelTapRows pixel_rows(const float* src, int C, int H, int W, int rows_h, int rows_w, int kh, int kw, int sh, int sw,
                               int ph, int pw, int rows) {
  PixelTapRows l;
  l.src = src; l.C = C; l.H = H; l.W = W;
  l.kh = kh; l.kw = kw; l.kwq = (kw + 3) / 4;
  l.sh = sh; l.sw = sw; l.ph = ph; l.pw = pw;
  l.rows = rows;
  l.d_hw.init(rows_h * rows_w);
  l.d_w.init(rows_w);
  l.d_kh.init(kh);
  l.d_kwq.init(l.kwq);
  return l;
}
inline TapWeights tap_weights(const float* w, int rows, int kh, int kw, int sn, int sc, int sky, int skx, int off0) {
  TapWeights l;
  l.w = w; l.rows = rows; l.kh = kh; l.kw = kw; l.kwq = (kw + 3) / 4;
  l.sn = sn; l.sc = sc; l.sky = sky; l.skx = skx; l.off0 = off0;
  l.d_kh.init(kh);
  l.d_kwq.init(l.kwq);
  return l;
}

}  // namespace tc

// Tensor-core GEMM with the rt_gemm contract.  Returns RT_ERR_UNIMPLEMENTED when the shape is
// not worth / not possible on this path, so that the caller can use the FP32 kernel.
rt_status rt_gemm_tc_internal(rt_ctx* ctx, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, const float* a,
                              int64_t lda, const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate) {
  using namespace tc;
  if (m <= 0 || n <= 0 || k <= 0) return RT_ERR_UNIMPLEMENTED;
  if (m >= (1ll << 31) || n >= (1ll << 31) || k >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  bool acc = accumulate != 0;
  if (use_ts_tile(ctx, m, n)) {
    const PlainA pa{a, lda, (int)m, trans_a != 0, al16(a) && lda % 4 == 0};
    if (!trans_b) return gemm_plain_ts(ctx, pa, MatMN{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
    return gemm_plain_ts(ctx, pa, MatK{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
  }
  // A(row=m, k): not transposed -> K-contiguous; transposed ([K,M] storage) -> M-contiguous
  // B(row=n, k): not transposed ([K,N] storage) -> N-contiguous; transposed ([N,K]) -> K-contiguous
  if (!trans_a && !trans_b)
    return gemm_plain(ctx, MatK{a, lda, (int)m, al16(a) && lda % 4 == 0}, MatMN{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
  if (!trans_a && trans_b)
    return gemm_plain(ctx, MatK{a, lda, (int)m, al16(a) && lda % 4 == 0}, MatK{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
  if (trans_a && !trans_b)
    return gemm_plain(ctx, MatMN{a, lda, (int)m, al16(a) && lda % 4 == 0}, MatMN{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
  return gemm_plain(ctx, MatMN{a, lda, (int)m, al16(a) && lda % 4 == 0}, MatK{b, ldb, (int)n, al16(b) && ldb % 4 == 0}, c, ldc, m, n, k, acc);
}

// y[Nb,Cy,Hy,Wy] = conv(x, w[Cy,Cx,kh,kw]) (+bias) on the tensor cores.
rt_status rt_conv_forward_tc_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g,
                                      float* y) {
  using namespace tc;
  int64_t M = (int64_t)g.Nb * g.Hy * g.Wy, N = g.Cy, K = (int64_t)g.Cx * g.kh * g.kw;
  if (M <= 0 || N <= 0 || K < 8 || M >= (1ll << 31) || (int64_t)g.Nb * g.Cx * g.Hx * g.Wx >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  ImageOut epi{y, bias, (int)N, g.Hy * g.Wy, (int)M, {}};
  epi.d_HW.init(g.Hy * g.Wy);
  if (g.kw <= 32) {  // padded-tap order: cheap pixel-row producer
    PixelTapRows la = pixel_rows(x, g.Cx, g.Hx, g.Wx, g.Hy, g.Wy, g.kh, g.kw, g.sh, g.sw, g.ph, g.pw, (int)M);
    TapWeights lb = tap_weights(w, (int)N, g.kh, g.kw, g.Cx * g.kh * g.kw, g.kh * g.kw, g.kw, 1, 0);
    const int Kp = g.Cx * g.kh * la.kwq * 4;
    return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, Kp, 1, (Kp + BK - 1) / BK * BK);
  }
  Im2colRows la{x, g, (int)M};
  MatK lb{w, K, (int)N, al16(w) && K % 4 == 0};
  return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, 1, (int)((K + BK - 1) / BK * BK));
}

// out[Nb,Cm,Hx,Wx] (+bias) = gather of y[Nb,Cy,Hy,Wy] with w[Cy,Cm,kh,kw] on the tensor cores
// (input gradient of a convolution; forward of a transposed convolution).
rt_status rt_conv_gather_tc_internal(rt_ctx* ctx, const float* y, const float* w, const float* bias, const ConvGeom& g,
                                     int cm, float* out) {
  using namespace tc;
  int64_t M = (int64_t)g.Nb * g.Hx * g.Wx, N = cm, K = (int64_t)g.Cy * g.kh * g.kw;
  if (M <= 0 || N <= 0 || K < 8 || M >= (1ll << 31) || (int64_t)g.Nb * g.Cy * g.Hy * g.Wy >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  ImageOut epi{out, bias, cm, g.Hx * g.Wx, (int)M, {}};
  epi.d_HW.init(g.Hx * g.Wx);
  if (g.sh == 1 && g.sw == 1 && g.kw <= 32) {
    // unit stride: the gather is a convolution of y with the kernel flipped in both directions and
    // padding (kh-1-ph, kw-1-pw), so the cheap pixel-row producer applies
    PixelTapRows la = pixel_rows(y, g.Cy, g.Hy, g.Wy, g.Hx, g.Wx, g.kh, g.kw, 1, 1, g.kh - 1 - g.ph, g.kw - 1 - g.pw, (int)M);
    TapWeights lb = tap_weights(w, cm, g.kh, g.kw, g.kh * g.kw, cm * g.kh * g.kw, -g.kw, -1, g.kh * g.kw - 1);
    const int Kp = g.Cy * g.kh * la.kwq * 4;
    return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, Kp, 1, (Kp + BK - 1) / BK * BK);
  }
  if ((g.sh > 1 || g.sw > 1) && g.kw <= 32 * g.sw) {
    // Strided gather (transposed-convolution forward, input gradient of a strided convolution): the outputs of one
    // stride phase (iy % sh, ix % sw) only meet the kernel taps ky = ky0 + sh*a, kx = kx0 + sw*b, and with those taps
    // the phase is a unit-stride convolution of y that writes every sh-th / sw-th output.  sh*sw launches without the
    // structural zeros replace one launch whose reduction is sh*sw times longer.
    bool ok = true;
    for (int ry = 0; ry < g.sh && ok; ++ry) ok = (ry + g.ph) % g.sh < g.kh || (g.Hx - ry + g.sh - 1) / g.sh <= 0;
    for (int rx = 0; rx < g.sw && ok; ++rx) ok = (rx + g.pw) % g.sw < g.kw || (g.Wx - rx + g.sw - 1) / g.sw <= 0;
    if (ok) {  // every non-empty phase has at least one tap (otherwise its outputs are the bias alone: generic path)
      for (int ry = 0; ry < g.sh; ++ry)
        for (int rx = 0; rx < g.sw; ++rx) {
          const int Hj = (g.Hx - ry + g.sh - 1) / g.sh, Wj = (g.Wx - rx + g.sw - 1) / g.sw;
          if (Hj <= 0 || Wj <= 0) continue;
          const int ky0 = (ry + g.ph) % g.sh, kx0 = (rx + g.pw) % g.sw;
          const int nay = (g.kh - ky0 + g.sh - 1) / g.sh, nax = (g.kw - kx0 + g.sw - 1) / g.sw;
          const int pt = (nay - 1) - (ry + g.ph - ky0) / g.sh, pl = (nax - 1) - (rx + g.pw - kx0) / g.sw;
          const int64_t Mp = (int64_t)g.Nb * Hj * Wj;
          PixelTapRows la = pixel_rows(y, g.Cy, g.Hy, g.Wy, Hj, Wj, nay, nax, 1, 1, pt, pl, (int)Mp);
          TapWeights lb = tap_weights(w, cm, nay, nax, g.kh * g.kw, cm * g.kh * g.kw, -g.sh * g.kw, -g.sw,
                                      (ky0 + g.sh * (nay - 1)) * g.kw + kx0 + g.sw * (nax - 1));
          PhaseOut pe{out, bias, cm, g.Hx, g.Wx, g.sh, g.sw, ry, rx, (int)Mp, {}, {}};
          pe.d_HjWj.init(Hj * Wj);
          pe.d_Wj.init(Wj);
          const int Kp = g.Cy * nay * la.kwq * 4;
          rt_status st = dispatch_bn(ctx, la, lb, pe, (int)Mp, (int)N, Kp, 1, (Kp + BK - 1) / BK * BK);
          if (st != RT_OK) return st;
        }
      return RT_OK;
    }
  }
  GatherRows la{y, g, (int)M};
  WeightSecondRows lb{w, g, cm};
  return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, 1, (int)((K + BK - 1) / BK * BK));
}

// dw[Cy, Cx*kh*kw] = sum over pixels of y * im2col(x) on the tensor cores.  The product is computed
// transposed (rows = taps, columns = Cy) so that the long side fills the 128-row tile, split along
// the pixel axis, written transposed into a workspace and summed deterministically.
rt_status rt_conv_weight_grad_tc_internal(rt_ctx* ctx, const float* x, const float* y, const ConvGeom& g, float* dw) {
  using namespace tc;
  int64_t M = (int64_t)g.Cx * g.kh * g.kw, N = g.Cy, K = (int64_t)g.Nb * g.Hy * g.Wy;
  if (M <= 0 || N <= 0 || K < 64 || K >= (1ll << 31) || (int64_t)g.Nb * g.Cx * g.Hx * g.Wx >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  int splits, kps;
  choose_split(ctx, M, N, K, &splits, &kps);
  // keep each accumulation chain short: at most 2048 reduction steps per split
  if (kps > 2048) {
    kps = 2048;
    splits = (int)((K + kps - 1) / kps);
  }
  Im2colK4 la{x, g, (int)M, g.sh * g.Wx - g.Wy * g.sw, (g.Cx * g.Hx - g.Hy * g.sh) * g.Wx};
  NarrowK4 lb{y, g, (int)N, al16(y) && (g.Hy * g.Wy) % 4 == 0};
  if (splits == 1) {
    TransposedOut epi{dw, M, 0, (int)M, (int)N};
    return dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, 1, kps);
  }
  RtScratch ws(ctx);
  rt_status st = ws.alloc(sizeof(float) * (size_t)splits * M * N);
  if (st != RT_OK) return st;
  TransposedOut epi{ws.as<float>(), M, M * N, (int)M, (int)N};
  st = dispatch_bn(ctx, la, lb, epi, (int)M, (int)N, (int)K, splits, kps);
  if (st != RT_OK) return st;
  return rt_sum_axis_internal(ctx, ws.as<float>(), 1, splits, M * N, dw, 1.f);
}
