// Integer helpers shared by the convolution kernels: division by run-time constants and the
// geometry of a convolution between a "wide" and a "narrow" NCHW tensor.
#pragma once
#include <cstdint>

// Division by a run-time constant through a multiply-high and a shift
// (valid for dividends below 2^31).
struct FastDiv {
  uint32_t d, mul, shr;
  void init(uint32_t div) {
    d = div;
    if (div <= 1) {
      mul = 0;
      shr = 0;
      return;
    }
    uint32_t l = 0;
    while ((1u << l) < div) ++l;
    uint32_t p = 31 + l;
    mul = (uint32_t)((((uint64_t)1 << p) + div - 1) / div);
    shr = p - 32;
  }
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d <= 1 ? n : (__umulhi(n, mul) >> shr); }
  __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};

// Geometry of a convolution between a "wide" tensor X[Nb, Cx, Hx, Wx] and a "narrow"
// tensor Y[Nb, Cy, Hy, Wy] with Hy = (Hx + 2*ph - kh)/sh + 1: y(b,cy,yo,xo) touches
// x(b,cx, yo*sh-ph+ky, xo*sw-pw+kx).
struct ConvGeom {
  int Nb, Cx, Hx, Wx, Cy, Hy, Wy, kh, kw, sh, sw, ph, pw;
  FastDiv d_khw, d_kw, d_HyWy, d_Wy, d_HxWx, d_Wx, d_sh, d_sw;
  void finish() {
    d_khw.init(kh * kw);
    d_kw.init(kw);
    d_HyWy.init(Hy * Wy);
    d_Wy.init(Wy);
    d_HxWx.init(Hx * Wx);
    d_Wx.init(Wx);
    d_sh.init(sh);
    d_sw.init(sw);
  }
};

inline ConvGeom make_geom(int64_t nb, int64_t cx, int64_t hx, int64_t wx, int64_t cy, int kh, int kw, int sh, int sw, int ph,
                   int pw) {
  ConvGeom g;
  g.Nb = (int)nb; g.Cx = (int)cx; g.Hx = (int)hx; g.Wx = (int)wx; g.Cy = (int)cy;
  g.kh = kh; g.kw = kw; g.sh = sh; g.sw = sw; g.ph = ph; g.pw = pw;
  g.Hy = (int)((hx + 2 * ph - kh) / sh + 1);
  g.Wy = (int)((wx + 2 * pw - kw) / sw + 1);
  g.finish();
  return g;
}

