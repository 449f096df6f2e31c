// Unit-stride convolution-shaped contractions on the tensor cores (tcgen05, 3xTF32) without an
// im2col expansion.  Used for conv2d forward, for the input gradient of conv2d and for the forward
// of conv2d_transpose when the stride is 1.
//
// The gathered tensor src[Nb,C,H,W] is viewed through its zero-padded "position space":
// position P = (b*Hp + yy)*Wp + xx with Hp = H+2ph, Wp = W+2pw.  The output pixel (b,y,x) sits at
// P = (b*Hp + y)*Wp + x and its tap (ky,kx) reads position P + ky*Wp + kx.  A CTA computes 128
// consecutive positions (the rows that are not output pixels - the padding columns and rows - are
// computed and dropped) and stages the window of positions they touch ONCE per channel group in
// shared memory, channels-last in groups of four: plane q holds channels 4q..4q+3, 16 bytes per
// position.  In the UMMA K-major core-matrix layout (8 rows x 16 bytes, rows 16 bytes apart, 8-row
// groups 128 bytes apart, K-chunks one plane apart) the operand of tap (ky,kx) is the same memory
// read from a start address shifted by (ky*Wp+kx)*16 bytes, so every staged element is split into
// hi / lo once and then used by all kh*kw taps: the CUDA cores do 1/(kh*kw) of the work of an
// im2col producer and the tensor cores set the pace.
//
// The weights are packed once per call by a small kernel into the exact shared-memory image
// (per tap a K-major [BN x Cp] tile, hi and lo) and stay resident in shared memory while the
// persistent CTA walks over its position tiles.  Roles per CTA: 8 producer / epilogue warps, one
// MMA-issuing thread.  Window stages and the two accumulator sets in tensor memory are handed
// over with mbarriers; every wait is bounded and on expiry the kernel records a code in the
// context's status word, skips the remaining work, frees its tensor memory and returns.
#include "rt_internal.cuh"
#include "conv_geom.cuh"
#include "tc_common.cuh"

namespace tc {
namespace conv {

constexpr int kProducerWarps = 8;
constexpr int kThreads = (kProducerWarps + 1) * 32;
constexpr int kTileM = 128;
// Accumulator columns per set: [hi*hi | hi*lo] (2*BN, one MMA against the stacked hi/lo weight tile) and lo*hi (BN).
// The reduction of one tile is at most a few hundred K-steps, short enough for a single accumulation chain.
constexpr int kAccCols = 3;
constexpr uint32_t kSmemLimit = 227 * 1024;
// after the window stages: 9 mbarriers, the tensor-memory address slot (16 bytes), 64 bias values
constexpr uint32_t kTmemSlotOffset = 9 * 8, kBiasOffset = kTmemSlotOffset + 16, kTailBytes = kBiasOffset + 64 * 4;
constexpr int kMaxCGQ = 8;  // channel quads per window stage held in registers by a producer thread

struct Params {
  const float* src;     // [Nb, C, H, W]
  const float* wimg;    // packed weights: hi image, then lo image
  const float* bias;    // per output channel or null
  float* out;           // [Nb, N, Ho, Wo]
  int Nb, C, H, W, Hp, Wp, ph, pw;
  int N, Ho, Wo, kh, kw;
  int NQ;               // channel quads in the padded channel count (even)
  int CGQ;              // channel quads per window stage (even)
  int groups;           // ceil(NQ / CGQ)
  int win;              // positions in a window, multiple of 8
  int tiles;            // ceil(Nb*Hp*Wp / 128)
  int wimg_floats;      // floats in one weight image (hi or lo): taps * BN * 4*NQ
  FastDiv d_HpWp, d_Wp;
};

// Packs w into the shared-memory image of the B operand: for tap t the K-major tile
// [2*BN rows x 4*NQ channels] (BN hi rows, then BN lo rows), core matrices of 8 rows x 4 channels, K-chunks 128 bytes apart,
// 8-row groups NQ*128 bytes apart.  value(n, c, t) = w[n*sn + c*sc + ky*sky + kx*skx + off0].
__global__ void pack_weights_kernel(const float* __restrict__ w, float* __restrict__ img, int N, int C, int BN, int NQ,
                                    int kh, int kw, int sn, int sc, int sky, int skx, int off0) {
  // The convolution kernel is launched as a programmatic dependent of this one: it may start its prologue (barriers, tensor
  // memory, the first window loads) right away and waits for this grid only before it fetches the packed weights.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int Cp = NQ * 4;
  const int per_tap = BN * Cp;
  const int total = kh * kw * per_tap;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int t = i / per_tap, r = i - t * per_tap;
    const int n = r / Cp, c = r - n * Cp;
    const int ky = t / kw, kx = t - ky * kw;
    float v = 0.f;
    if (n < N && c < C) v = __ldg(w + n * sn + c * sc + ky * sky + kx * skx + off0);
    const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const int dst = t * 2 * per_tap + (n >> 3) * (NQ * 32) + (c >> 2) * 32 + (n & 7) * 4 + (c & 3);
    img[dst] = hi;
    img[per_tap + dst] = v - hi;  // the lo tile follows the hi tile of the same tap: together a 2*BN-row operand
  }
}

// CGQ = channel quads per window stage (2, 4, 6 or 8), a compile-time constant so that the producers' load / convert /
// store loops are straight-line code: these nine warps are issue-bound, every predicate and address computation in the
// per-element path shows up in the kernel's run time.
template <int BN, int CGQ>
__global__ void __launch_bounds__(kThreads, 1) conv_window_kernel(const Params p, int* status) {
  extern __shared__ __align__(128) char smem[];
  constexpr uint32_t kTmemCols = BN == 32 ? 256 : 512;  // two accumulator sets of 3*BN columns, rounded to a power of two
  static_assert(2 * kAccCols * BN <= kTmemCols, "accumulator sets must fit the allocation");
  // The warp index and the tensor-memory base are broadcast from lane 0: a value that comes out of a shuffle from a fixed lane is
  // known to be the same in every lane, so the role branches are uniform and the MMA warp's descriptor arithmetic can stay in
  // uniform registers, which is where tcgen05.mma takes its operands from.
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int taps = p.kh * p.kw;
  const uint32_t plane = (uint32_t)p.win * 16;               // bytes of one channel-quad plane
  const uint32_t a_half = (uint32_t)CGQ * plane;           // hi (or lo) part of a window stage
  const uint32_t a_stage = 2 * a_half;
  const uint32_t b_half = (uint32_t)p.wimg_floats * 4;       // hi (or lo) weight image
  const uint32_t tap_bytes = 2u * BN * p.NQ * 16;            // one tap: hi tile + lo tile
  // shared memory: weights (hi, lo) | window stage 0 | window stage 1 | barriers | tmem slot
  const uint32_t off_a = 2 * b_half;
  const uint32_t off_bar = off_a + 2 * a_stage;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bars = smem_base + off_bar;  // a_full[2], a_empty[2], acc_full[2], acc_empty[2], b_full
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bar + kTmemSlotOffset);
  float* bias_s = reinterpret_cast<float*>(smem + off_bar + kBiasOffset);  // BN <= 64 floats

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bars + 8 * s, kProducerWarps);        // a_full
      mbar_init(bars + 8 * (2 + s), 1);               // a_empty
      mbar_init(bars + 8 * (4 + s), 1);               // acc_full
      mbar_init(bars + 8 * (6 + s), kProducerWarps);  // acc_empty
    }
    mbar_init(bars + 8 * 8, 1);                       // b_full: the resident weights have landed
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kProducerWarps) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  if (threadIdx.x < BN) bias_s[threadIdx.x] = (p.bias && (int)threadIdx.x < p.N) ? __ldg(p.bias + threadIdx.x) : 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  const int my_tiles = p.tiles > (int)blockIdx.x ? (p.tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  bool ok = true;

  if (warp < kProducerWarps) {
    // ---------------- window producers, then epilogue of the previous tile ----------------
    const int tid = threadIdx.x;  // position within the window (threads beyond the window idle in the producer part)
    const int hw = p.H * p.W;
    auto epilogue = [&](int tile, int tcnt) -> bool {
      const int set = tcnt & 1;
      if (!mbar_wait(bars + 8 * (4 + set), (tcnt >> 1) & 1, status, 5)) return false;
      tc_fence_after();
      const int quad = warp & 3, half = warp >> 2;
      const int P = tile * kTileM + quad * 32 + lane;
      uint32_t b, r, y, x;
      p.d_HpWp.divmod(P, b, r);
      p.d_Wp.divmod(r, y, x);
      const bool valid = (int)b < p.Nb && (int)y < p.Ho && (int)x < p.Wo;
      const int howo = p.Ho * p.Wo;
      float* q = p.out + (int64_t)b * p.N * howo + (int)y * p.Wo + (int)x;
      // this warp's share: 32 rows (its lane quadrant) x BN/2 columns, in pieces of 16 columns
      constexpr int CW = BN / 2;
#pragma unroll
      for (int c0 = 0; c0 < CW; c0 += 16) {
        const int col = half * CW + c0;
        const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(set * kAccCols * BN + col);
        uint32_t r[kAccCols][16];
#pragma unroll
        for (int a = 0; a < kAccCols; ++a) tmem_ld16_nowait(t0 + (uint32_t)(a * BN), r[a]);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = col + j;
            const float v = __uint_as_float(r[0][j]) + (__uint_as_float(r[1][j]) + __uint_as_float(r[2][j]));
            if (n < p.N) q[(int64_t)n * howo] = v + bias_s[n];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (6 + set));
      return true;
    };

    // A stage is (tile, channel group).  The loads of stage s+1 are issued before stage s is converted
    // and stored, so that their latency overlaps the wait for the stage buffer and the conversion.
    struct Pos { bool inside; int soff; };
    auto decode = [&](int i) -> Pos {  // this thread's window position in the i-th tile of this CTA
      Pos ps{false, 0};
      if (tid < p.win) {
        const int P = ((int)blockIdx.x + i * (int)gridDim.x) * kTileM + tid;
        uint32_t b, r, yy, xx;
        p.d_HpWp.divmod(P, b, r);
        p.d_Wp.divmod(r, yy, xx);
        const int y = (int)yy - p.ph, x = (int)xx - p.pw;
        ps.inside = (int)b < p.Nb && (unsigned)y < (unsigned)p.H && (unsigned)x < (unsigned)p.W;
        ps.soff = ((int)b * p.C * p.H + y) * p.W + x;
      }
      return ps;
    };
    struct Buf { float v[CGQ][4]; };
    auto load = [&](const Pos& ps, int g, Buf& bf) {
      const int c00 = g * CGQ * 4;
      if (ps.inside && c00 + CGQ * 4 <= p.C) {  // the common case: a whole group of real channels, no per-element tests
        const float* src = p.src + ps.soff + c00 * hw;
#pragma unroll
        for (int q = 0; q < CGQ; ++q)
#pragma unroll
          for (int j = 0; j < 4; ++j) bf.v[q][j] = __ldg(src + (q * 4 + j) * hw);
      } else {
#pragma unroll
        for (int q = 0; q < CGQ; ++q)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c00 + q * 4 + j;
            bf.v[q][j] = (ps.inside && c < p.C) ? __ldg(p.src + ps.soff + c * hw) : 0.f;
          }
      }
    };
    auto store = [&](int scnt, int g, const Buf& bf) -> bool {
      const int slot = scnt & 1;
      if (scnt >= 2 && !mbar_wait(bars + 8 * (2 + slot), ((scnt >> 1) - 1) & 1, status, 4)) return false;
      if (tid < p.win) {
        char* a_hi = smem + off_a + slot * a_stage + (uint32_t)tid * 16;
        char* a_lo = a_hi + a_half;
        const int nq = min(CGQ, p.NQ - g * CGQ);
#pragma unroll
        for (int q = 0; q < CGQ; ++q)
          if (q < nq) {
            float4 vh, vl;
            split4(bf.v[q], vh, vl);
            *reinterpret_cast<float4*>(a_hi + (uint32_t)q * plane) = vh;
            *reinterpret_cast<float4*>(a_lo + (uint32_t)q * plane) = vl;
          }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * slot);
      return true;
    };
    const int total = my_tiles * p.groups;
    Buf b0, b1;
    Pos ps = decode(0);
    int ti = 0, g = 0;  // tile / group of the stage whose data sits in the "current" buffer
    if (total > 0) load(ps, 0, b0);
    // one step: prefetch the next stage into `nxt`, then convert and store `cur`
    auto step = [&](int s, const Buf& cur, Buf& nxt) -> bool {
      int nti = ti, ng = g + 1;
      if (ng == p.groups) { ng = 0; ++nti; }
      if (s + 1 < total) {
        if (nti != ti) ps = decode(nti);
        load(ps, ng, nxt);
      }
      if (!store(s, g, cur)) return false;
      if (g == p.groups - 1 && ti > 0 && !epilogue((int)blockIdx.x + (ti - 1) * (int)gridDim.x, ti - 1)) return false;
      ti = nti;
      g = ng;
      return true;
    };
    for (int s = 0; s < total && ok; s += 2) {
      ok = step(s, b0, b1);
      if (ok && s + 1 < total) ok = step(s + 1, b1, b0);
    }
    if (ok && my_tiles > 0) ok = epilogue((int)blockIdx.x + (my_tiles - 1) * (int)gridDim.x, my_tiles - 1);
  } else {
    // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
    // Descriptors are kept as 32-bit low words (start address, in 16-byte units, plus the constant
    // leading-dimension field) that advance by additions; the issue loop has no divisions.
    constexpr uint32_t idesc_n = make_idesc(BN), idesc_2n = make_idesc(2 * BN);
    const uint32_t a_hi32 = desc_hi32(128), b_hi32 = desc_hi32((uint32_t)p.NQ * 128);
    const uint32_t a_kstep = (2 * plane) >> 4, b_kstep = 256 >> 4;   // two channel quads per K-step
    const uint32_t a_lo_delta = a_half >> 4;  // hi window -> lo window
    const uint32_t tap_step = tap_bytes >> 4;
    // resident weights: bulk copies of the packed image, in pieces of at most 32 KiB
    {
      const uint32_t bytes = 2 * b_half;
      asm volatile("griddepcontrol.wait;" ::: "memory");  // the packing kernel has finished and its image is visible
      if (lane == 0) {
        mbar_expect_tx(bars + 8 * 8, bytes);
        for (uint32_t o = 0; o < bytes; o += 32768u) {
          const uint32_t n = bytes - o < 32768u ? bytes - o : 32768u;
          bulk_copy_g2s(smem_base + o, reinterpret_cast<const char*>(p.wimg) + o, n, bars + 8 * 8);
        }
      }
      __syncwarp();
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * 8, 0, status, 8));
    }
    int scnt = 0;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int set = i & 1;
      if (i >= 2) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (6 + set), ((i >> 1) - 1) & 1, status, 6));
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + (uint32_t)(set * kAccCols * BN);
      uint32_t first = 0;  // becomes 1 after the first K-step of the tile
      for (int g = 0; g < p.groups && ok; ++g, ++scnt) {
        const int slot = scnt & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * slot, (scnt >> 1) & 1, status, 7));
        if (!ok) break;
        tc_fence_after();
        const int q0 = g * CGQ;
        const int nk = min(CGQ, p.NQ - q0) >> 1;  // K-steps of 8 channels
        const uint32_t a_base = desc_lo32(smem_base + off_a + slot * a_stage, plane);
        uint32_t b_tap = desc_lo32(smem_base + (uint32_t)q0 * 128, 128);
        for (int ky = 0; ky < p.kh; ++ky) {
          uint32_t a_tap = a_base + (uint32_t)(ky * p.Wp);
          for (int kx = 0; kx < p.kw; ++kx, ++a_tap, b_tap += tap_step) {
            uint32_t a = a_tap, b = b_tap;
            for (int j = 0; j < nk; ++j, a += a_kstep, b += b_kstep) {
              umma_tf32_pair_elect(acc, acc + 2 * BN, a, a + a_lo_delta, a_hi32, b, b_hi32, idesc_2n, idesc_n, first);
              first = 1;
            }
          }
        }
        umma_commit_elect(bars + 8 * (2 + slot));  // the window stage may be refilled once these MMAs have read it
      }
      if (ok) umma_commit_elect(bars + 8 * (4 + set));  // accumulator set complete
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace conv
}  // namespace tc

// out[Nb,N,Ho,Wo] (+bias) = sum over (c,ky,kx) of src[b,c,y-ph+ky,x-pw+kx] * W(n,c,ky,kx), unit stride, with
// W(n,c,ky,kx) = w[n*sn + c*sc + ky*sky + kx*skx + off0].  Returns RT_ERR_UNIMPLEMENTED when the shape does not
// fit this kernel (more than 64 output channels, weights that do not fit in shared memory, ...).
rt_status rt_conv_window_tc_internal(rt_ctx* ctx, const float* src, int Nb, int C, int H, int W, int ph, int pw, const float* w,
                                     int N, int kh, int kw, int sn, int sc, int sky, int skx, int off0, const float* bias,
                                     float* out) {
  using namespace tc;
  using namespace tc::conv;
  if (ph < 0 || pw < 0 || N < 1 || N > 64 || C < 1 || Nb < 1) return RT_ERR_UNIMPLEMENTED;
  const int Hp = H + 2 * ph, Wp = W + 2 * pw;
  const int Ho = Hp - kh + 1, Wo = Wp - kw + 1;
  if (Ho < 1 || Wo < 1) return RT_ERR_UNIMPLEMENTED;
  const int64_t positions = (int64_t)Nb * Hp * Wp;
  if (positions + kTileM >= (1ll << 31) || (int64_t)Nb * C * H * W >= (1ll << 31) || (int64_t)Nb * N * Ho * Wo >= (1ll << 31))
    return RT_ERR_UNIMPLEMENTED;
  const int BN = N <= 32 ? 32 : 64;
  Params p{};
  p.src = src; p.bias = bias; p.out = out;
  p.Nb = Nb; p.C = C; p.H = H; p.W = W; p.Hp = Hp; p.Wp = Wp; p.ph = ph; p.pw = pw;
  p.N = N; p.Ho = Ho; p.Wo = Wo; p.kh = kh; p.kw = kw;
  p.NQ = ((C + 7) / 8) * 2;
  p.win = (kTileM + (kh - 1) * Wp + (kw - 1) + 7) / 8 * 8;
  if (p.win > 8 * 32) return RT_ERR_UNIMPLEMENTED;  // one producer thread per window position
  p.tiles = (int)((positions + kTileM - 1) / kTileM);
  p.wimg_floats = kh * kw * BN * p.NQ * 4;
  const uint32_t b_bytes = 2u * (uint32_t)p.wimg_floats * 4u;
  const uint32_t plane = (uint32_t)p.win * 16;
  if (plane > 262128u || (uint32_t)p.NQ * 128u > 262128u) return RT_ERR_UNIMPLEMENTED;
  // fewest channel groups whose two window stages fit next to the resident weights
  p.CGQ = 0;
  for (int groups = 1; groups <= p.NQ / 2; ++groups) {
    int cgq = (p.NQ + groups - 1) / groups;
    cgq += cgq & 1;
    const uint64_t need = (uint64_t)b_bytes + 2ull * 2 * cgq * plane + kTailBytes;
    if (cgq <= kMaxCGQ && need <= kSmemLimit) {
      p.CGQ = cgq;
      break;
    }
  }
  if (p.CGQ == 0) return RT_ERR_UNIMPLEMENTED;
  p.groups = (p.NQ + p.CGQ - 1) / p.CGQ;
  p.d_HpWp.init(Hp * Wp);
  p.d_Wp.init(Wp);
  const uint32_t smem_bytes = b_bytes + 2u * 2u * (uint32_t)p.CGQ * plane + kTailBytes;

  RtScratch wimg(ctx);
  rt_status st = wimg.alloc(b_bytes);
  if (st != RT_OK) return st;
  p.wimg = wimg.as<float>();
  pack_weights_kernel<<<rt_grid_for(ctx, p.wimg_floats, 256), 256, 0, ctx->stream>>>(w, wimg.as<float>(), N, C, BN, p.NQ, kh, kw, sn,
                                                                                    sc, sky, skx, off0);
  RT_LAUNCHED(ctx);
  const int grid = p.tiles < ctx->sm_count ? p.tiles : ctx->sm_count;
  auto launch = [&](auto kern) -> rt_status {
    RT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    RT_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p, ctx->device_status));
    return RT_OK;
  };
  rt_status ls;
  if (BN == 32) {
    ls = p.CGQ == 2 ? launch(conv_window_kernel<32, 2>) : p.CGQ == 4 ? launch(conv_window_kernel<32, 4>)
       : p.CGQ == 6 ? launch(conv_window_kernel<32, 6>) : launch(conv_window_kernel<32, 8>);
  } else {
    ls = p.CGQ == 2 ? launch(conv_window_kernel<64, 2>) : p.CGQ == 4 ? launch(conv_window_kernel<64, 4>)
       : p.CGQ == 6 ? launch(conv_window_kernel<64, 6>) : launch(conv_window_kernel<64, 8>);
  }
  if (ls != RT_OK) return ls;
  RT_LAUNCHED(ctx);
  return RT_OK;
}
