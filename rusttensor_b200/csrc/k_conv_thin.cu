// Convolutions whose reduction is tiny (Cin*kh*kw <= 16 taps, e.g. the first layer of a CNN on
// single-channel images): a GEMM formulation would fill a tile with zeros, so these run as direct
// FP32 kernels.  A thread owns one output pixel and keeps its taps in registers.
//   forward:          y[b,n,p] = bias[n] + sum_t tap_t(b,p) * w[n,t]
//   weight gradient:  dw[n,t]  = sum_{b,p} g[b,n,p] * tap_t(b,p)   (per-warp partial sums over a pixel
//                     range, then a deterministic second pass; single-channel 3x3 layers: whole images per block, with db)
//   forward fused with bias + relu + 2x2 max pooling for single-channel 3x3 layers
// tap_t(b,p) = x[b, c, yo*sh-ph+ky, xo*sw-pw+kx] for t = (c,ky,kx), zero outside the image.
#include "rt_internal.cuh"
#include "conv_geom.cuh"

rt_status rt_sum_axis_internal(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* out,
                               float scale);

namespace {

constexpr int kMaxTaps = 16;
constexpr int kThreads = 256;

struct ThinParams {
  const float* x;   // [Nb, C, H, W]
  int Nb, C, H, W, N, Ho, Wo, sh, sw;
  int T;            // C*kh*kw
  int64_t pixels;   // Nb*Ho*Wo
  FastDiv d_HoWo, d_Wo;
  int dy[kMaxTaps], dx[kMaxTaps], off[kMaxTaps];  // tap t: row / column displacement and c*H*W + dy*W + dx
};

// Reads the TP taps of output pixel (b, yo, xo); entries t >= T are zero.
template <int TP>
__device__ __forceinline__ void load_taps(const ThinParams& p, uint32_t b, uint32_t yo, uint32_t xo, float (&tap)[TP]) {
  const int y0 = (int)yo * p.sh, x0 = (int)xo * p.sw;
  const float* base = p.x + ((int64_t)b * p.C * p.H + y0) * p.W + x0;
#pragma unroll
  for (int t = 0; t < TP; ++t) {
    const bool in = t < p.T && (unsigned)(y0 + p.dy[t]) < (unsigned)p.H && (unsigned)(x0 + p.dx[t]) < (unsigned)p.W;
    tap[t] = in ? __ldg(base + p.off[t]) : 0.f;
  }
}

// Thread = output pixel: its taps sit in registers, the weights in shared memory transposed to [tap][channel] so that one
// 128-bit broadcast load brings a tap's weights for four channels.  Four channels are computed at a time - four independent
// chains of fused multiply-adds, each in the order bias, then the taps (ky, kx) ascending - and stored as four coalesced rows.
// NQC > 0: the layer has exactly 4 * NQC output channels, a compile-time constant, so that the channel loop unrolls into
// straight-line code with immediate shared-memory offsets and no tests (the kernel is bound by instruction issue: the
// run-time loop spent 1 100 instructions per warp on 288 fused multiply-adds per lane).  NQC == 0: any channel count.
template <int TP, int NQC>
__global__ void __launch_bounds__(kThreads) thin_conv_forward_kernel(const ThinParams p, const float* __restrict__ w,
                                                                      const float* __restrict__ bias, float* __restrict__ y) {
  extern __shared__ __align__(16) float sm[];  // w_t[TP][NP], bias_s[NP]; NP = N rounded up to a multiple of four
  const int NP = NQC > 0 ? 4 * NQC : (p.N + 3) & ~3;
  float* w_t = sm;
  float* bias_s = sm + TP * NP;
  // the taps of the first pixel are requested before the weights are staged, so that the two latencies overlap
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t px = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  uint32_t b = 0, r = 0, yo, xo;
  float tap[TP];
  if (px < p.pixels) {
    p.d_HoWo.divmod((uint32_t)px, b, r);
    p.d_Wo.divmod(r, yo, xo);
    load_taps<TP>(p, b, yo, xo, tap);
  }
  for (int i = threadIdx.x; i < TP * NP; i += kThreads) {
    const int t = i / NP, n = i - t * NP;
    w_t[i] = (t < p.T && n < p.N) ? __ldg(w + n * p.T + t) : 0.f;
  }
  for (int i = threadIdx.x; i < NP; i += kThreads) bias_s[i] = (bias && i < p.N) ? __ldg(bias + i) : 0.f;
  __syncthreads();
  const int howo = p.Ho * p.Wo;
  while (px < p.pixels) {
    float* out = y + (int64_t)b * p.N * howo + r;
    if (NQC > 0) {
#pragma unroll
      for (int q = 0; q < NQC; ++q) {
        float4 acc = *reinterpret_cast<const float4*>(bias_s + 4 * q);
#pragma unroll
        for (int t = 0; t < TP; ++t) {
          const float4 wv = *reinterpret_cast<const float4*>(w_t + t * (4 * NQC) + 4 * q);
          acc.x = fmaf(tap[t], wv.x, acc.x);
          acc.y = fmaf(tap[t], wv.y, acc.y);
          acc.z = fmaf(tap[t], wv.z, acc.z);
          acc.w = fmaf(tap[t], wv.w, acc.w);
        }
        out[0] = acc.x;
        out[howo] = acc.y;
        out[2 * howo] = acc.z;
        out[3 * howo] = acc.w;
        out += 4 * howo;
      }
    } else {
      for (int n = 0; n < p.N; n += 4) {
        float4 acc = *reinterpret_cast<const float4*>(bias_s + n);
#pragma unroll
        for (int t = 0; t < TP; ++t) {
          const float4 wv = *reinterpret_cast<const float4*>(w_t + t * NP + n);
          acc.x = fmaf(tap[t], wv.x, acc.x);
          acc.y = fmaf(tap[t], wv.y, acc.y);
          acc.z = fmaf(tap[t], wv.z, acc.z);
          acc.w = fmaf(tap[t], wv.w, acc.w);
        }
        float* o = out + (int64_t)n * howo;
        o[0] = acc.x;
        if (n + 1 < p.N) o[howo] = acc.y;
        if (n + 2 < p.N) o[2 * (int64_t)howo] = acc.z;
        if (n + 3 < p.N) o[3 * (int64_t)howo] = acc.w;
      }
    }
    px += stride;
    if (px < p.pixels) {
      p.d_HoWo.divmod((uint32_t)px, b, r);
      p.d_Wo.divmod(r, yo, xo);
      load_taps<TP>(p, b, yo, xo, tap);
    }
  }
}

// One block per range of 512 output pixels.  Phase 1: every thread gathers the taps of two pixels (all
// loads in flight at once) into shared memory, together with the offset of the pixel in g.  Phase 2:
// warp w owns output channels w*4 .. w*4+3 (+32, +64, ...): lane = pixel, 4 x TP accumulators per lane
// fed from shared memory, reduced over the lanes at the end.  part[range][n][t], t < T.
constexpr int kRangePixels = 512;
template <int TP>
__global__ void __launch_bounds__(kThreads) thin_conv_dw_kernel(const ThinParams p, const float* __restrict__ g,
                                                                 float* __restrict__ part) {
  __shared__ float taps_s[TP][kRangePixels];
  __shared__ int goff_s[kRangePixels];  // b*N*Ho*Wo + pixel-in-image, or -1 past the end
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int howo = p.Ho * p.Wo;
  const int64_t p0 = (int64_t)blockIdx.x * kRangePixels;
#pragma unroll
  for (int h = 0; h < kRangePixels / kThreads; ++h) {
    const int i = threadIdx.x + h * kThreads;
    const int64_t px = p0 + i;
    float tap[TP];
    int go = -1;
    if (px < p.pixels) {
      uint32_t b, r, yo, xo;
      p.d_HoWo.divmod((uint32_t)px, b, r);
      p.d_Wo.divmod(r, yo, xo);
      load_taps<TP>(p, b, yo, xo, tap);
      go = (int)b * p.N * howo + (int)r;
    } else {
#pragma unroll
      for (int t = 0; t < TP; ++t) tap[t] = 0.f;
    }
#pragma unroll
    for (int t = 0; t < TP; ++t) taps_s[t][i] = tap[t];
    goff_s[i] = go;
  }
  __syncthreads();
  for (int n0 = warp * 4; n0 < p.N; n0 += (kThreads / 32) * 4) {
    float acc[4][TP];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int t = 0; t < TP; ++t) acc[i][t] = 0.f;
    constexpr int kUnroll = 4;
    for (int k0 = 0; k0 < kRangePixels / 32; k0 += kUnroll) {
      float gv[kUnroll][4];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int go = goff_s[(k0 + u) * 32 + lane];
#pragma unroll
        for (int i = 0; i < 4; ++i) gv[u][i] = (go >= 0 && n0 + i < p.N) ? __ldg(g + go + (int64_t)(n0 + i) * howo) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int t = 0; t < TP; ++t) {
          const float tv = taps_s[t][(k0 + u) * 32 + lane];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][t] = fmaf(gv[u][i], tv, acc[i][t]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int t = 0; t < TP; ++t) {
        float v = acc[i][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && n0 + i < p.N && t < p.T) part[((int64_t)blockIdx.x * p.N + n0 + i) * p.T + t] = v;
      }
  }
}

// ---- weight and bias gradient of a single-channel, unit-stride convolution, whole images per block ----------------
// dw[n, ky, kx] = sum_{b, yo, xo} g[b, n, yo, xo] * x[b, yo - ph + ky, xo - pw + kx],  db[n] = sum g[b, n, :, :].
// A block walks over images b = blockIdx.x, blockIdx.x + gridDim.x, ...: the image, with its zero halo, sits in shared
// memory (the next one is fetched into registers meanwhile); warps w and w + 8 own output channels 4w .. 4w+3 of the current
// group of 32 and take alternate blocks of 128 output pixels, their lanes stride over the pixels with coalesced loads of g
// (the next block's loads in flight while the current one is accumulated), and the 4 x (KH*KW + 1) running sums stay in
// registers across all images of the block.  One pass over g yields dw and db.  The per-block sums are added in a fixed
// order by a two-level hand-over: the block that arrives last in its group of eight adds the group's partial sums, the
// group that arrives last adds the groups' - whichever blocks these happen to be, the order of the additions is the same.
struct ImageDwParams {
  const float* x;  // [Nb, 1, H, W]
  const float* g;  // [Nb, N, Ho, Wo]
  float* part1;    // [gridDim.x][N * (T + 1)]
  float* part2;    // [groups][N * (T + 1)]
  float* dw;       // [N, T]
  float* db;       // [N] or null
  unsigned* tickets;  // [1 + groups], zero between launches
  int Nb, H, W, N, Ho, Wo, ph, pw, Hp, Wp;
  FastDiv d_Wo, d_Wp, d_Wq;  // d_Wq: Wo / 4 (pixel quads per output row)
};
constexpr int kGroupBlocks = 8;

constexpr int kImgThreads = 512;

// QUAD (Wo a multiple of 4, KW odd): a lane takes four horizontally adjacent pixels at a time - one 128-bit load of g per channel
// and the KH x (KW + 3) patch of the image as 64-bit shared-memory loads - which halves the instructions per multiply-add.
template <int KH, int KW, bool QUAD>
__global__ void __launch_bounds__(kImgThreads) thin_dw_image_kernel(const ImageDwParams p) {
  constexpr int T = KH * KW;
  extern __shared__ __align__(16) float tile[];  // Hp x Wp: the image with its halo
  __shared__ float phase1[8][4][T + 1];          // sums of the warps that took the odd pixel blocks
  __shared__ int is_last;
  // warp = (pixel phase, channel quad): warps w and w + 8 share four output channels and take alternate blocks of 128 pixels
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = warp & 7, phase = warp >> 3;
  const int howo = p.Ho * p.Wo, tile_n = p.Hp * p.Wp, outs = p.N * (T + 1);
  constexpr int kPre = 2;  // halo tile elements a thread carries for the next image (more: a second round after the swap)
  auto fetch = [&](int b, int i) -> float {
    uint32_t ty, tx;
    p.d_Wp.divmod((uint32_t)i, ty, tx);
    const int iy = (int)ty - p.ph, ix = (int)tx - p.pw;
    return ((unsigned)iy < (unsigned)p.H && (unsigned)ix < (unsigned)p.W) ? __ldg(p.x + ((int64_t)b * p.H + iy) * p.W + ix) : 0.f;
  };
  for (int c0 = 0; c0 < p.N; c0 += 32) {
    const int n0 = c0 + quad * 4;
    float acc[4][T + 1];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int t = 0; t <= T; ++t) acc[i][t] = 0.f;
    __syncthreads();  // the tile of the previous channel group is no longer read
    for (int i = threadIdx.x; i < tile_n; i += kImgThreads) tile[i] = fetch(blockIdx.x, i);
    __syncthreads();
    for (int b = blockIdx.x; b < p.Nb; b += gridDim.x) {
      const int nb = b + gridDim.x;
      float pre[kPre];
#pragma unroll
      for (int u = 0; u < kPre; ++u) {
        const int i = threadIdx.x + u * kImgThreads;
        pre[u] = (nb < p.Nb && i < tile_n) ? fetch(nb, i) : 0.f;
      }
      const float* gb = p.g + ((int64_t)b * p.N + n0) * howo;
      if constexpr (QUAD) {
        // the gradients of the next pixel quads are in flight while the current ones are accumulated
        const int nquads = howo >> 2;
        float4 gv[4], gn[4];
        auto load_q = [&](int qd, float4 (&dst)[4]) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = (qd < nquads && n0 + i < p.N) ? __ldg(reinterpret_cast<const float4*>(gb + (int64_t)i * howo) + qd)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        load_q(phase * 32 + lane, gv);
        for (int base = phase * 32; base < nquads; base += 64) {
          const int qd = base + lane;
          load_q(qd + 64, gn);
          uint32_t yo, xq;
          p.d_Wq.divmod(qd < nquads ? (uint32_t)qd : 0u, yo, xq);
          const float2* tp = reinterpret_cast<const float2*>(tile + (int)yo * p.Wp + 4 * (int)xq);  // Wp and 4*xq are even
          float pt[KH][KW + 3];
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int j = 0; j < (KW + 3) / 2; ++j) {
              const float2 t2 = tp[(ky * p.Wp >> 1) + j];
              pt[ky][2 * j] = t2.x;
              pt[ky][2 * j + 1] = t2.y;
            }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float gq[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w};
#pragma unroll
            for (int d = 0; d < 4; ++d)
#pragma unroll
              for (int ky = 0; ky < KH; ++ky)
#pragma unroll
                for (int kx = 0; kx < KW; ++kx) acc[i][ky * KW + kx] = fmaf(gq[d], pt[ky][d + kx], acc[i][ky * KW + kx]);
            acc[i][T] += (gq[0] + gq[1]) + (gq[2] + gq[3]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) gv[i] = gn[i];
        }
      } else {
      // the gradients of the next block of pixels are in flight while the current one is accumulated
      float gv[4][4], gn[4][4];
      auto load_g = [&](int q0, float (&dst)[4][4]) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int q = q0 + u * 32 + lane;
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[u][i] = (q < howo && n0 + i < p.N) ? __ldg(gb + (int64_t)i * howo + q) : 0.f;
        }
      };
      load_g(phase * 128, gv);
      for (int q0 = phase * 128; q0 < howo; q0 += 256) {
        load_g(q0 + 256, gn);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int q = q0 + u * 32 + lane;
          uint32_t yo, xo;
          p.d_Wo.divmod(q < howo ? (uint32_t)q : 0u, yo, xo);
          const float* tp = tile + (int)yo * p.Wp + (int)xo;
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int kx = 0; kx < KW; ++kx) {
              const float tv = tp[ky * p.Wp + kx];
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[i][ky * KW + kx] = fmaf(gv[u][i], tv, acc[i][ky * KW + kx]);
            }
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][T] += gv[u][i];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int i = 0; i < 4; ++i) gv[u][i] = gn[u][i];
      }
      }
      __syncthreads();  // every warp is done with this image
      if (nb < p.Nb) {
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
          const int i = threadIdx.x + u * kImgThreads;
          if (i < tile_n) tile[i] = pre[u];
        }
        for (int i = threadIdx.x + kPre * kImgThreads; i < tile_n; i += kImgThreads) tile[i] = fetch(nb, i);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int t = 0; t <= T; ++t) {
        float v = acc[i][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[i][t] = v;
      }
    if (phase == 1 && lane == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int t = 0; t <= T; ++t) phase1[quad][i][t] = acc[i][t];
    }
    __syncthreads();
    if (phase == 0 && lane == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int t = 0; t <= T; ++t)
          if (n0 + i < p.N) p.part1[(int64_t)blockIdx.x * outs + (n0 + i) * (T + 1) + t] = acc[i][t] + phase1[quad][i][t];
    }
  }
  // level 1: the last block of each group of eight adds the group's partial sums
  const int grp = blockIdx.x / kGroupBlocks, groups = (gridDim.x + kGroupBlocks - 1) / kGroupBlocks;
  const int gsize = min(kGroupBlocks, (int)gridDim.x - grp * kGroupBlocks);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    is_last = atomicAdd(p.tickets + 1 + grp, 1u) == (unsigned)gsize - 1;
    if (is_last) p.tickets[1 + grp] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int o = threadIdx.x; o < outs; o += kImgThreads) {
    float v[kGroupBlocks];
#pragma unroll
    for (int j = 0; j < kGroupBlocks; ++j) v[j] = j < gsize ? __ldcg(p.part1 + (int64_t)(grp * kGroupBlocks + j) * outs + o) : 0.f;
    float sum = v[0];
#pragma unroll
    for (int j = 1; j < kGroupBlocks; ++j) sum += v[j];
    p.part2[(int64_t)grp * outs + o] = sum;
  }
  // level 2: the last group adds the groups' sums and writes the result
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    is_last = atomicAdd(p.tickets, 1u) == (unsigned)groups - 1;
    if (is_last) p.tickets[0] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int o = threadIdx.x; o < outs; o += kImgThreads) {
    float sum = 0.f;
    int j = 0;
    for (; j + 8 <= groups; j += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(p.part2 + (int64_t)(j + u) * outs + o);
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += v[u];
    }
    for (; j < groups; ++j) sum += __ldcg(p.part2 + (int64_t)j * outs + o);
    const int n = o / (T + 1), t = o - n * (T + 1);
    if (t < T) p.dw[n * T + t] = sum;
    else if (p.db) p.db[n] = sum;
  }
}

// ---- conv2d (single channel, 3x3, unit stride) + bias + relu + 2x2/stride-2 max pooling in one pass ----------------------
// A thread owns one pooled pixel and a group of 16 output channels: it reads the 4x4 input patch its 2x2 window of
// convolution outputs touches once, and for every channel forms the four outputs with the SAME sequence of fused multiply-adds
// as thin_conv_forward_kernel (bias first, then the taps in (ky, kx) order), applies relu and keeps the first maximum in window
// order - so values and indices are bit-identical to conv2d -> relu -> max_pool2d, and the convolution output never exists.
struct ThinPoolParams {
  const float* x;  // [Nb, 1, H, W]
  int Nb, H, W, N, Hp, Wp, ph, pw;  // Hp x Wp: the pooled extent (convolution output Ho = 2*Hp, Wo = 2*Wp)
  int64_t pooled;                   // Nb * Hp * Wp
  FastDiv d_HpWp, d_Wp;
};
constexpr int kPoolChannelGroup = 16;

__global__ void __launch_bounds__(kThreads) thin_conv_relu_pool_kernel(const ThinPoolParams p, const float* __restrict__ w,
                                                                        const float* __restrict__ bias, float* __restrict__ y,
                                                                        float* __restrict__ idx) {
  // weights transposed to [tap][channel]: one 128-bit broadcast load brings a tap's weights for four channels; channels past the
  // layer's last one hold zeros and are computed but not stored
  __shared__ __align__(16) float w_t[9][kPoolChannelGroup];
  __shared__ __align__(16) float b_s[kPoolChannelGroup];
  const int n0 = blockIdx.y * kPoolChannelGroup;
  const int nn = min(kPoolChannelGroup, p.N - n0);
  for (int i = threadIdx.x; i < kPoolChannelGroup * 9; i += kThreads) {
    const int n = i / 9, t = i - n * 9;
    w_t[t][n] = n < nn ? __ldg(w + (n0 + n) * 9 + t) : 0.f;
  }
  for (int i = threadIdx.x; i < kPoolChannelGroup; i += kThreads) b_s[i] = (bias && i < nn) ? __ldg(bias + n0 + i) : 0.f;
  __syncthreads();
  const int hpwp = p.Hp * p.Wp;
  for (int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x; q < p.pooled; q += (int64_t)gridDim.x * kThreads) {
    uint32_t b, r, yp, xp;
    p.d_HpWp.divmod((uint32_t)q, b, r);
    p.d_Wp.divmod(r, yp, xp);
    float patch[4][4];
    const int y0 = 2 * (int)yp - p.ph, x0 = 2 * (int)xp - p.pw;
    const float* img = p.x + (int64_t)b * p.H * p.W;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int iy = y0 + i, ix = x0 + j;
        patch[i][j] = ((unsigned)iy < (unsigned)p.H && (unsigned)ix < (unsigned)p.W) ? __ldg(img + iy * p.W + ix) : 0.f;
      }
    float* yo = y + ((int64_t)b * p.N + n0) * hpwp + r;
    float* io = idx + ((int64_t)b * p.N + n0) * hpwp + r;
#pragma unroll
    for (int c4 = 0; c4 < kPoolChannelGroup; c4 += 4) {
      if (c4 < nn) {  // the same for every thread of the block
        // acc[d][j]: output d of the 2x2 window (row-major) for channel c4 + j; per output the chain is bias, then the taps in
        // (ky, kx) order - the order of thin_conv_forward_kernel
        float acc[4][4];
        const float4 bv = *reinterpret_cast<const float4*>(&b_s[c4]);
#pragma unroll
        for (int d = 0; d < 4; ++d) { acc[d][0] = bv.x; acc[d][1] = bv.y; acc[d][2] = bv.z; acc[d][3] = bv.w; }
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
          for (int kx = 0; kx < 3; ++kx) {
            const float4 wv = *reinterpret_cast<const float4*>(&w_t[ky * 3 + kx][c4]);
#pragma unroll
            for (int d = 0; d < 4; ++d) {
              const float a = patch[(d >> 1) + ky][(d & 1) + kx];
              acc[d][0] = fmaf(a, wv.x, acc[d][0]);
              acc[d][1] = fmaf(a, wv.y, acc[d][1]);
              acc[d][2] = fmaf(a, wv.z, acc[d][2]);
              acc[d][3] = fmaf(a, wv.w, acc[d][3]);
            }
          }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (c4 + j < nn) {
            float mv = -INFINITY;
            int mi = 0;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
              const float v = fmaxf(acc[d][j], 0.f);
              if (v > mv) { mv = v; mi = d; }
            }
            yo[(int64_t)(c4 + j) * hpwp] = mv;
            io[(int64_t)(c4 + j) * hpwp] = (float)mi;
          }
        }
      }
    }
  }
}

bool make_params(const ConvGeom& g, const float* x, ThinParams* p) {
  const int T = g.Cx * g.kh * g.kw;
  const int64_t pixels = (int64_t)g.Nb * g.Hy * g.Wy;
  if (T < 1 || T > kMaxTaps || pixels < 1 || pixels >= (1ll << 31) || (int64_t)g.Cx * g.Hx * g.Wx >= (1ll << 30)) return false;
  p->x = x;
  p->Nb = g.Nb; p->C = g.Cx; p->H = g.Hx; p->W = g.Wx; p->N = g.Cy; p->Ho = g.Hy; p->Wo = g.Wy; p->sh = g.sh; p->sw = g.sw;
  p->T = T;
  p->pixels = pixels;
  p->d_HoWo.init(g.Hy * g.Wy);
  p->d_Wo.init(g.Wy);
  for (int t = 0; t < kMaxTaps; ++t) p->dy[t] = p->dx[t] = p->off[t] = 0;
  int t = 0;
  for (int c = 0; c < g.Cx; ++c)
    for (int ky = 0; ky < g.kh; ++ky)
      for (int kx = 0; kx < g.kw; ++kx, ++t) {
        p->dy[t] = ky - g.ph;
        p->dx[t] = kx - g.pw;
        p->off[t] = (c * g.Hx + ky - g.ph) * g.Wx + kx - g.pw;
      }
  return true;
}

}  // namespace

// y = conv2d(x, w) + bias for Cx*kh*kw <= 16; RT_ERR_UNIMPLEMENTED otherwise.
rt_status rt_conv_forward_thin_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g,
                                        float* y) {
  ThinParams p;
  if (g.Cy < 1 || g.Cy > 512 || !make_params(g, x, &p)) return RT_ERR_UNIMPLEMENTED;
  const int TP = p.T == 9 ? 9 : (p.T + 3) / 4 * 4;  // a 3x3 single-channel layer gets its exact tap count
  const int NP = (g.Cy + 3) & ~3;
  const size_t smem = sizeof(float) * (size_t)(NP * TP + NP);
  const int grid = rt_grid_for(ctx, p.pixels, kThreads, 16);
  if ((int64_t)g.Cy * p.Ho * p.Wo >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;  // channel offsets inside one image are 32-bit
  switch (TP) {
    case 9:
      if (g.Cy == 16) thin_conv_forward_kernel<9, 4><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y);
      else if (g.Cy == 32) thin_conv_forward_kernel<9, 8><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y);
      else if (g.Cy == 64) thin_conv_forward_kernel<9, 16><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y);
      else thin_conv_forward_kernel<9, 0><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y);
      break;
    case 4: thin_conv_forward_kernel<4, 0><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y); break;
    case 8: thin_conv_forward_kernel<8, 0><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y); break;
    case 12: thin_conv_forward_kernel<12, 0><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y); break;
    default: thin_conv_forward_kernel<16, 0><<<grid, kThreads, smem, ctx->stream>>>(p, w, bias, y); break;
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// y, idx = max_pool2d(relu(conv2d(x, w) + bias), 2x2, stride 2) for a single-channel 3x3 unit-stride convolution with an even
// output extent; RT_ERR_UNIMPLEMENTED otherwise.
rt_status rt_conv_relu_pool_thin_internal(rt_ctx* ctx, const float* x, const float* w, const float* bias, const ConvGeom& g, float* y,
                                          float* idx) {
  if (g.Cx != 1 || g.kh != 3 || g.kw != 3 || g.sh != 1 || g.sw != 1 || g.Hy < 2 || g.Wy < 2 || (g.Hy & 1) || (g.Wy & 1) || g.Cy < 1)
    return RT_ERR_UNIMPLEMENTED;
  ThinPoolParams p;
  p.x = x; p.Nb = g.Nb; p.H = g.Hx; p.W = g.Wx; p.N = g.Cy; p.Hp = g.Hy / 2; p.Wp = g.Wy / 2; p.ph = g.ph; p.pw = g.pw;
  p.pooled = (int64_t)g.Nb * p.Hp * p.Wp;
  if (p.pooled < 1 || p.pooled >= (1ll << 31) || (int64_t)g.Nb * g.Cy * p.Hp * p.Wp >= (1ll << 40)) return RT_ERR_UNIMPLEMENTED;
  p.d_HpWp.init(p.Hp * p.Wp);
  p.d_Wp.init(p.Wp);
  const int groups = (g.Cy + kPoolChannelGroup - 1) / kPoolChannelGroup;
  if (groups > 65535) return RT_ERR_UNIMPLEMENTED;
  const dim3 grid(rt_grid_for(ctx, p.pooled, kThreads, 16), groups);
  thin_conv_relu_pool_kernel<<<grid, kThreads, 0, ctx->stream>>>(p, w, bias, y, idx);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// The single-channel whole-image kernel: unit stride, 3x3 window, the image with its halo within 48 KB of shared memory.
static rt_status weight_grad_image(rt_ctx* ctx, const float* x, const float* gy, const ConvGeom& g, float* dw, float* db) {
  if (g.Cx != 1 || g.sh != 1 || g.sw != 1 || g.kh != 3 || g.kw != 3 || g.Cy < 1 || g.Nb < 1 || !ctx->reduce_counters)
    return RT_ERR_UNIMPLEMENTED;
  ImageDwParams p;
  p.Hp = g.Hy + g.kh - 1;
  p.Wp = g.Wy + g.kw - 1;
  const size_t smem = sizeof(float) * (size_t)p.Hp * p.Wp;
  if (g.Hy < 1 || g.Wy < 1 || smem > 48 * 1024 || (int64_t)g.Nb * g.Cy * g.Hy * g.Wy >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  const int T = g.kh * g.kw, outs = g.Cy * (T + 1);
  const int grid = g.Nb < ctx->sm_count ? g.Nb : ctx->sm_count;
  const int groups = (grid + kGroupBlocks - 1) / kGroupBlocks;
  if (1 + groups > kAuxCounterSlots) return RT_ERR_UNIMPLEMENTED;
  RtScratch part(ctx);
  rt_status st = part.alloc(sizeof(float) * (size_t)(grid + groups) * outs);
  if (st != RT_OK) return st;
  p.x = x; p.g = gy; p.dw = dw; p.db = db;
  p.part1 = part.as<float>();
  p.part2 = p.part1 + (size_t)grid * outs;
  p.tickets = ctx->reduce_counters + 2 * kReduceCounterSlots + (ctx->on_side ? kAuxCounterSlots : 0);
  p.Nb = g.Nb; p.H = g.Hx; p.W = g.Wx; p.N = g.Cy; p.Ho = g.Hy; p.Wo = g.Wy; p.ph = g.ph; p.pw = g.pw;
  p.d_Wo.init(g.Wy);
  p.d_Wp.init(p.Wp);
  p.d_Wq.init(g.Wy / 4 > 0 ? g.Wy / 4 : 1);
  if (g.Wy % 4 == 0 && rt_aligned16(gy)) thin_dw_image_kernel<3, 3, true><<<grid, kImgThreads, smem, ctx->stream>>>(p);
  else thin_dw_image_kernel<3, 3, false><<<grid, kImgThreads, smem, ctx->stream>>>(p);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// dw[Cy, Cx*kh*kw] = sum over pixels of g * im2col(x) for Cx*kh*kw <= 16; RT_ERR_UNIMPLEMENTED otherwise.  With `db` not null
// the bias gradient db[Cy] may come out of the same pass; *db_done tells whether it did.
rt_status rt_conv_weight_grad_thin_internal(rt_ctx* ctx, const float* x, const float* gy, const ConvGeom& g, float* dw, float* db,
                                            bool* db_done) {
  if (db_done) *db_done = false;
  {
    const rt_status st = weight_grad_image(ctx, x, gy, g, dw, db_done ? db : nullptr);
    if (st == RT_OK && db && db_done) *db_done = true;
    if (st != RT_ERR_UNIMPLEMENTED) return st;
  }
  ThinParams p;
  if (g.Cy < 1 || !make_params(g, x, &p)) return RT_ERR_UNIMPLEMENTED;
  const int TP = (p.T + 3) / 4 * 4;
  const int ranges = (int)((p.pixels + kRangePixels - 1) / kRangePixels);
  RtScratch part(ctx);
  float* dst = dw;
  if (ranges > 1) {
    rt_status st = part.alloc(sizeof(float) * (size_t)ranges * g.Cy * p.T);
    if (st != RT_OK) return st;
    dst = part.as<float>();
  }
  if ((int64_t)g.Nb * g.Cy * g.Hy * g.Wy >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  switch (TP) {
    case 4: thin_conv_dw_kernel<4><<<ranges, kThreads, 0, ctx->stream>>>(p, gy, dst); break;
    case 8: thin_conv_dw_kernel<8><<<ranges, kThreads, 0, ctx->stream>>>(p, gy, dst); break;
    case 12: thin_conv_dw_kernel<12><<<ranges, kThreads, 0, ctx->stream>>>(p, gy, dst); break;
    default: thin_conv_dw_kernel<16><<<ranges, kThreads, 0, ctx->stream>>>(p, gy, dst); break;
  }
  RT_LAUNCHED(ctx);
  if (ranges > 1) return rt_sum_axis_internal(ctx, dst, 1, ranges, (int64_t)g.Cy * p.T, dw, 1.f);
  return RT_OK;
}
