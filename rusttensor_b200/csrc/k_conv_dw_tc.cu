// Weight gradient of a unit-stride convolution on the tensor cores (tcgen05, 3xTF32), fed by TMA, with the
// reduction running over output pixels:
//
//   dw[co, ci, ky, kx] = sum over (b, yo, xo) of  g[b, co, yo, xo] * x[b, ci, yo - ph + ky, xo - pw + kx]
//   db[co]             = sum over (b, yo, xo) of  g[b, co, yo, xo]                       (optional, same pass over g)
//
// No im2col matrix exists, not even in shared memory.  The unit of work is one output row segment (b, yo, columns
// c0 .. c0+SW): its P (8, 16 or 32) pixels are the K index of the MMAs.
//   A operand (M = 128 rows): the 64 output channels of the CTA's tile, split into hi (rows 0..63) and lo (rows 64..127),
//     K = the P pixels of the row segment.  It lives in TENSOR MEMORY: converter threads read the TMA-staged g row,
//     split it and write it with tcgen05.st, so the MMA reads only the B operand from shared memory (an MMA whose A
//     operand comes from shared memory is bound by shared-memory bandwidth: 32 + N/4 cycles instead of N/2).
//   B operand (N = kw * CIT rows): for every kernel column kx the CIT input channels of the CTA's tile, K = pixels of ONE
//     input row shifted by kx.  A window row is converted once (kw shifted images, hi and lo) into a ring in shared
//     memory and then used by the kh output rows that touch it: the kernel-row offset ky is simply "which ring slot".
//   D (kh accumulators of N columns, fp32, tensor memory): D_ky[r, kx*CIT + ci] += A[r, :] . B_row(yo-ph+ky)[kx*CIT+ci, :].
//     Both the hi and the lo image of B are multiplied into the same accumulator, so rows 0..63 hold g_hi * x and rows
//     64..127 g_lo * x; the epilogue adds the two halves.
// Rows of g and x reach shared memory through cp.async.bulk.tensor (TMA, 3-D maps over [HW, C, N], every CTA fetching its own rows) issued by
// one thread several stages ahead; eight converter warps turn them into MMA operands; one warp issues the MMAs.  The CTAs
// of one (output-channel tile, input-channel tile) pair split the units among themselves; every CTA writes its partial
// sums to a workspace and a second kernel adds the partials in a fixed order (bit-reproducible, no atomics).  Long
// reductions are cut into segments of at most ~1024 accumulations per accumulator, each flushed as a partial of its own:
// the tensor core adds into the fp32 accumulator with truncation, an error that grows with the length of the chain.
//
// Every wait is bounded; on expiry the kernel records a code in the context's status word, raises a CTA-wide abort flag
// that every other wait polls, frees its tensor memory and returns.
#include <cuda.h>

#include "conv_geom.cuh"
#include "rt_internal.cuh"
#include "tc_common.cuh"

namespace tc {
namespace dw {

constexpr int kConvWarps = 16;                     // converter / epilogue warps
constexpr int kGroupWarps = 8, kGroupThreads = kGroupWarps * 32;  // warps 0..7 convert x rows, warps 8..15 convert g rows
constexpr int kThreads = (kConvWarps + 2) * 32;    // + TMA warp + MMA warp
constexpr int kCoTile = 64;
constexpr int RG = 3, RX = 3;                      // ring depths: raw g boxes, raw x boxes
constexpr int kMaxDA = 8;                          // A slots in tensor memory (2 * group size)
constexpr int kMaxDB = 12, kMaxKh = 5, kMaxKw = 4;
constexpr uint32_t kTmemCols = 512;
constexpr int kNumBars = 2 * RG + 2 * RX + 2 * kMaxDA + 2 * kMaxDB + 2;

struct Params {
  float* ws;      // [n_combo][cpc*SEG][64][kh][kw][CIT] partial weight gradients (the accumulators' own column order)
  float* ws_db;   // [n_cot][cpc][64] partial bias gradients (tiles with cit == 0), or null
  int Nb, Cin, Cout, H, W, Ho, Wo, kh, kw, ph, pw;
  int nseg, SW;   // column segments per row, segment width (<= P)
  int CIT, N;     // input channels per tile, N = kw * CIT
  int n_cot, n_cit, n_combo, cpc, SEG;
  int units;      // Nb * nseg * Ho
  int BWg, BWx;   // TMA box widths (floats), 4 * odd
  int DB;         // depth of the window-row ring
  int R;          // units the MMA warp issues back to back (one round of waits and commits per group)
  int GL, RB;     // units per g box / window rows per x box: R when the units of a strip are contiguous in memory (one
                  // column segment per row), else 1.  The TMA unit spends its time per box ROW (one contiguous run per
                  // channel), about 26 cycles each, so the runs are made as long as the layout allows.
  int DA, da_shift;  // A slots in tensor memory (a power of two, 2 * R), log2
  int row_len;    // CIT * kh * kw
  uint32_t off_raw_x, off_b, off_bar;  // shared memory offsets (raw g rows start at 0)
  uint32_t raw_g_bytes, raw_x_bytes, b_img_bytes;
  FastDiv d_Ho, d_nseg;
};

// ---- small PTX helpers --------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem descriptor]; one elected lane of a converged warp issues.
__device__ __forceinline__ void umma_ts_elect(uint32_t d, uint32_t a_tmem, uint32_t b_lo32, uint32_t b_hi32, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred pa, pe;\n\t"
      ".reg .b64 db;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, pa;\n\t}" ::"r"(d), "r"(a_tmem), "r"(b_lo32), "r"(b_hi32),
      "r"(idesc), "r"(accumulate)
      : "memory");
}
// Bounded wait that also gives up when another role of the CTA has already failed.
// Bounded wait that also gives up when another role of the CTA has already failed.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  // try_wait suspends the thread in hardware for a bounded time, so the loop polls without sleeping for a long while
  // (a sleeping waiter adds its wake-up latency to every hand-over of the pipeline) and backs off only when something
  // is clearly stuck.
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
    if (i > 8192) __nanosleep(256);
  }
  record_status(status, code);
  *abort_flag = 1;
  return false;
}

// A run = consecutive units of one column strip (b, seg) inside one segment: output rows y0 .. y_end-1.  Every role walks
// the same runs; inside a run the window rows are consecutive ring events, and each run loads its own rows.
struct Run {
  int b, c0, swv, y0, y_end;
  __device__ __forceinline__ Run(const Params& p, int u, int s_end) {
    uint32_t ss, yy, bb, sg;
    p.d_Ho.divmod((uint32_t)u, ss, yy);
    p.d_nseg.divmod(ss, bb, sg);
    b = (int)bb;
    c0 = (int)sg * p.SW;
    swv = min(p.SW, p.Wo - c0);
    y0 = (int)yy;
    y_end = min(p.Ho, y0 + (s_end - u));
  }
};
// Position in the window-row ring: slot, parity of the number of wraps, "has wrapped".
struct RingPos {
  int pos = 0;
  uint32_t par = 0;
  bool wrapped = false;
  __device__ __forceinline__ void advance(int depth) {
    if (++pos == depth) { pos = 0; par ^= 1u; wrapped = true; }
  }
};

// a = hi + lo with hi = a with the low 13 mantissa bits cleared
__device__ __forceinline__ float hi_part(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

// NC pixels of one row of g (one output channel, from the TMA-staged copy) -> one lane of the A slot in tensor memory:
// hi rows get the value with the low mantissa bits cleared, lo rows the remainder.  `mask` bit c = pixel c belongs to
// the segment.  Returns the sum of the row (for the bias gradient).
template <int NC, int OFF>
__device__ __forceinline__ float convert_g_row(const float* raw_row, uint32_t mask, int part, uint32_t taddr) {
  float c[NC + 4];
  const float4* src = reinterpret_cast<const float4*>(raw_row);
#pragma unroll
  for (int m = 0; m < NC / 4 + 1; ++m) {
    const float4 t = src[m];
    c[4 * m] = t.x; c[4 * m + 1] = t.y; c[4 * m + 2] = t.z; c[4 * m + 3] = t.w;
  }
  float sum = 0.f;
#pragma unroll
  for (int j0 = 0; j0 < NC; j0 += 4) {
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float v = (mask >> (j0 + j)) & 1u ? c[OFF + j0 + j] : 0.f;
      sum += v;
      const float h = hi_part(v);
      out[j] = __float_as_uint(part == 0 ? h : v - h);
    }
    tmem_st4(taddr + (uint32_t)j0, out);
  }
  return sum;
}

// Four pixels of one input channel of a window row -> the kw shifted K-chunks of the B operand (hi and lo image).
// `src` points at the 16-byte chunk that holds the first source element, `mask` bit i = source column of element i lies
// inside the image, dst = chunk of kernel column 0, `step` = bytes between kernel columns.
template <int OFF>
__device__ __forceinline__ void convert_x_item(const float* src, uint32_t mask, int kw, char* dst, uint32_t step, uint32_t img_bytes) {
  float c[12];
#pragma unroll
  for (int m = 0; m < 3; ++m) {
    const float4 t = reinterpret_cast<const float4*>(src)[m];
    c[4 * m] = t.x; c[4 * m + 1] = t.y; c[4 * m + 2] = t.z; c[4 * m + 3] = t.w;
  }
  float eh[4 + kMaxKw - 1], el[4 + kMaxKw - 1];
#pragma unroll
  for (int i = 0; i < 4 + kMaxKw - 1; ++i) {
    const float v = (mask >> i) & 1u ? c[OFF + i] : 0.f;
    eh[i] = hi_part(v);
    el[i] = v - eh[i];
  }
#pragma unroll
  for (int kx = 0; kx < kMaxKw; ++kx) {
    if (kx < kw) {
      *reinterpret_cast<float4*>(dst + kx * step) = make_float4(eh[kx], eh[kx + 1], eh[kx + 2], eh[kx + 3]);
      *reinterpret_cast<float4*>(dst + kx * step + img_bytes) = make_float4(el[kx], el[kx + 1], el[kx + 2], el[kx + 3]);
    }
  }
}

// Both MMAs of one K-step (B hi image, then B lo image) into the same accumulator; one elected lane issues.
__device__ __forceinline__ void umma_ts_pair_elect(uint32_t d, uint32_t a_tmem, uint32_t b_hi_img, uint32_t b_lo_img, uint32_t b_hi32,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred pa, pe, pt;\n\t"
      ".reg .b64 d1, d2;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %6, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 d1, {%2, %4};\n\t"
      "mov.b64 d2, {%3, %4};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d1, %5, pa;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d2, %5, pt;\n\t}" ::"r"(d), "r"(a_tmem), "r"(b_hi_img), "r"(b_lo_img),
      "r"(b_hi32), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int P>
__global__ void __launch_bounds__(kThreads, 1)
conv_dw_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x, const Params p, int* status) {
  extern __shared__ __align__(128) char smem[];
  constexpr int KSTEPS = P / 8;
  // broadcast from lane 0 so that the compiler knows the value is the same in every lane (uniform role branches and registers)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int combo = (int)blockIdx.x % p.n_combo, slot_id = (int)blockIdx.x / p.n_combo;
  const int cot = combo / p.n_cit, cit = combo - cot * p.n_cit;
  // this CTA's units, cut into SEG segments
  const int per = (p.units + p.cpc - 1) / p.cpc;
  const int u_begin = min(p.units, slot_id * per), u_end = min(p.units, u_begin + per);
  const int seg_len = (u_end - u_begin + p.SEG - 1) / p.SEG;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bars = smem_base + p.off_bar;
  const uint32_t bar_gf = bars, bar_ge = bar_gf + 8 * RG, bar_xf = bar_ge + 8 * RG, bar_xe = bar_xf + 8 * RX;
  const uint32_t bar_af = bar_xe + 8 * RX, bar_ae = bar_af + 8 * kMaxDA, bar_bf = bar_ae + 8 * kMaxDA, bar_be = bar_bf + 8 * kMaxDB;
  const uint32_t bar_df = bar_be + 8 * kMaxDB, bar_de = bar_df + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + p.off_bar + kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* started_word = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);
  float* db_scratch = reinterpret_cast<float*>(tmem_slot + 4);  // 64 floats: bias-gradient sums of the second pixel half
  bool db_half0 = false;
  float db_value = 0.f;
  int db_channel = 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RG; ++s) { mbar_init(bar_gf + 8 * s, 1); mbar_init(bar_ge + 8 * s, kGroupWarps); }
    for (int s = 0; s < RX; ++s) { mbar_init(bar_xf + 8 * s, 1); mbar_init(bar_xe + 8 * s, kGroupWarps); }
    for (int s = 0; s < kMaxDA; ++s) { mbar_init(bar_af + 8 * s, kGroupWarps); mbar_init(bar_ae + 8 * s, 1); }
    for (int s = 0; s < kMaxDB; ++s) { mbar_init(bar_bf + 8 * s, kGroupWarps); mbar_init(bar_be + 8 * s, 1); }
    mbar_init(bar_df, 1);
    mbar_init(bar_de, kConvWarps);
    *abort_flag = 0;
    *started_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kConvWarps + 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  const uint32_t a_col0 = (uint32_t)(p.kh * p.N);  // the A slots follow the kh accumulators

  if (warp == kConvWarps) {
    // ---------------------------------------------- TMA thread ----------------------------------------------
    if (lane == 0) {
      bool ok = true;
      int gi = 0, e = 0;  // g boxes / x boxes so far
      for (int sg = 0; sg < p.SEG && ok; ++sg) {
        const int s_begin = min(u_end, u_begin + sg * seg_len), s_end = min(u_end, s_begin + seg_len);
        for (int u = s_begin; u < s_end && ok;) {
          const Run r(p, u, s_end);
          int next_row = max(0, r.y0 - p.ph);
          for (int yo = r.y0; yo < r.y_end && ok;) {  // one group of units at a time, as the MMA warp takes them
            const int rn = min(p.R, r.y_end - yo);
            const int top = min(p.H - 1, yo + rn - 1 - p.ph + p.kh - 1);
            while (next_row <= top && ok) {            // x boxes: the window rows this group adds
              const int nb = min(p.RB, top + 1 - next_row), s = e % RX;
              if (e >= RX) ok = wait_bar(bar_xe + 8 * s, ((e / RX) - 1) & 1, status, 31, abort_flag);
              if (!ok) break;
              const int e0 = next_row * p.W + r.c0 - p.pw;
              mbar_expect_tx(bar_xf + 8 * s, p.raw_x_bytes);
              tma_load_3d(smem_base + p.off_raw_x + (uint32_t)s * p.raw_x_bytes, &map_x, (e0 >> 2) << 2, cit * p.CIT, r.b, bar_xf + 8 * s);
              next_row += nb;
              ++e;
            }
            for (int k0 = 0; k0 < rn && ok; k0 += p.GL, ++gi) {  // g boxes: the rows of this group's units
              const int s = gi % RG;
              if (gi >= RG) ok = wait_bar(bar_ge + 8 * s, ((gi / RG) - 1) & 1, status, 32, abort_flag);
              if (!ok) break;
              const int e0 = (yo + k0) * p.Wo + r.c0;
              mbar_expect_tx(bar_gf + 8 * s, p.raw_g_bytes);
              tma_load_3d(smem_base + (uint32_t)s * p.raw_g_bytes, &map_g, e0 & ~3, cot * kCoTile, r.b, bar_gf + 8 * s);
            }
            yo += rn;
          }
          u += r.y_end - r.y0;
        }
      }
    }
  } else if (warp == kConvWarps + 1) {
    // ---------------------------------------------- MMA warp ------------------------------------------------
    const uint32_t idesc = make_idesc(p.N);
    const uint32_t b_hi32 = desc_hi32((uint32_t)P * 32);
    const uint32_t b_slot_units = (2 * p.b_img_bytes) >> 4, b_img_units = p.b_img_bytes >> 4;
    const uint32_t b_ring = desc_lo32(smem_base + p.off_b, 128);
    RingPos ring;       // next event to arrive
    int live_slot = 0;  // ring slot of the lowest live row (rows are released in the order they were produced)
    bool ok = true;
    int i = 0;
    for (int sg = 0; sg < p.SEG && ok; ++sg) {
      const int s_begin = min(u_end, u_begin + sg * seg_len), s_end = min(u_end, s_begin + seg_len);
      if (sg > 0) {
        ok = __all_sync(0xffffffffu, wait_bar(bar_de, (sg - 1) & 1, status, 33, abort_flag));
        if (!ok) break;
        tc_fence_after();
      }
      uint32_t started = 0;
      for (int u = s_begin; u < s_end && ok;) {
        const Run r(p, u, s_end);
        int next_row = max(0, r.y0 - p.ph), live_lo = next_row;
        // Groups of up to R units: one round of waits, then all their MMAs back to back, then the commits - the
        // tensor pipe idles while this warp waits and commits, so that part is paid once per group.
        for (int yo = r.y0; yo < r.y_end && ok;) {
          const int rn = min(p.R, r.y_end - yo);
          const int top = min(p.H - 1, yo + rn - 1 - p.ph + p.kh - 1);
          for (; next_row <= top && ok; ++next_row) {
            ok = __all_sync(0xffffffffu, wait_bar(bar_bf + 8 * ring.pos, ring.par, status, 34, abort_flag));
            ring.advance(p.DB);
          }
          for (int k = 0; k < rn && ok; ++k) {
            const int sa = (i + k) & (p.DA - 1);
            ok = __all_sync(0xffffffffu, wait_bar(bar_af + 8 * sa, ((i + k) >> p.da_shift) & 1, status, 35, abort_flag));
          }
          if (!ok) break;
          tc_fence_after();
          for (int k = 0; k < rn; ++k) {
            const int y = yo + k, sa = (i + k) & (p.DA - 1);
            const uint32_t a_t = tmem_base + a_col0 + (uint32_t)(sa * P);
            // the rows of the window are consecutive events: the slot of a row follows from its distance to the lowest live row
            const int ky_lo = max(0, p.ph - y), ky_hi = min(p.kh, p.H + p.ph - y);
            int slot = live_slot + (y - p.ph + ky_lo - live_lo);
            if (slot >= p.DB) slot -= p.DB;
            uint32_t d = tmem_base + (uint32_t)(ky_lo * p.N);
            for (int ky = ky_lo; ky < ky_hi; ++ky, d += (uint32_t)p.N) {
              const uint32_t b0 = b_ring + (uint32_t)slot * b_slot_units;
              umma_ts_pair_elect(d, a_t, b0, b0 + b_img_units, b_hi32, idesc, (started >> ky) & 1u);
#pragma unroll
              for (int j = 1; j < KSTEPS; ++j) umma_ts_pair_elect(d, a_t + 8 * j, b0 + 16 * j, b0 + b_img_units + 16 * j, b_hi32, idesc, 1u);
              started |= 1u << ky;
              if (++slot == p.DB) slot = 0;
            }
            umma_commit_elect(bar_ae + 8 * sa);
          }
          for (; live_lo < min(next_row, yo + rn - p.ph); ++live_lo) {  // rows above the next group's window are dead now
            umma_commit_elect(bar_be + 8 * live_slot);
            if (++live_slot == p.DB) live_slot = 0;
          }
          yo += rn;
          i += rn;
        }
        for (; live_lo < next_row; ++live_lo) {  // end of the run: the rows still live are released (the next run loads its own)
          umma_commit_elect(bar_be + 8 * live_slot);
          if (++live_slot == p.DB) live_slot = 0;
        }
        u += r.y_end - r.y0;
      }
      if (!ok) break;
      if (lane == 0) {
        *started_word = started;
        __threadfence_block();
      }
      __syncwarp();
      umma_commit_elect(bar_df);
    }
  } else {
    // ------------------- converters: warps 0..3 window rows of x, warps 4..7 rows of g; all eight: epilogue ---------
    const int tid = threadIdx.x;
    const bool x_group = warp < kGroupWarps;
    // q: quarter of the tensor-memory lanes this warp may touch; half: which half of a row's pixels a g converter takes;
    // cgrp: which of four interleaved sets of accumulator chunks the warp stores in the epilogue
    const int q = warp & 3, half = (warp >> 2) & 1, cgrp = warp >> 2;
    // A rows are interleaved: tensor-memory lane 2c holds the hi part of channel c, lane 2c+1 its lo part
    const int part = lane & 1;
    const int co_l = q * 16 + (lane >> 1);           // output channel within the tile
    const uint32_t t_lane = (uint32_t)(32 * q) << 16;
    float db_acc = 0.f;
    bool ok = true;
    int i = 0, e = 0;
    RingPos ring;
    // per-thread constants of the x items (at most two per thread: CIT <= 32, P <= 32, 256 threads)
    const uint32_t sbo = (uint32_t)P * 32, kx_step = (uint32_t)(p.CIT >> 3) * sbo;
    int it_c4[2], it_src[2];
    uint32_t it_dst[2], it_mask[2] = {0u, 0u};
    const int x_items = p.CIT * (P / 4);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int it = tid + k * kGroupThreads;
      const int c4 = it / p.CIT, ci = it - c4 * p.CIT;
      it_c4[k] = it < x_items ? c4 : -1;
      it_src[k] = ci * p.BWx + 4 * c4;
      it_dst[k] = (uint32_t)(ci >> 3) * sbo + (uint32_t)c4 * 128 + (uint32_t)(ci & 7) * 16;
    }
    for (int sg = 0; sg < p.SEG && ok; ++sg) {
      const int s_begin = min(u_end, u_begin + sg * seg_len), s_end = min(u_end, s_begin + seg_len);
      for (int u = s_begin; u < s_end && ok;) {
        const Run r(p, u, s_end);
        if (x_group) {
          // source-column masks of this strip: bit i = the column of element i lies inside the image
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int cs0 = r.c0 - p.pw + 4 * it_c4[k];
            uint32_t m = 0;
#pragma unroll
            for (int b2 = 0; b2 < 4 + kMaxKw - 1; ++b2) m |= ((unsigned)(cs0 + b2) < (unsigned)p.W ? 1u : 0u) << b2;
            it_mask[k] = m;
          }
          int next_row = max(0, r.y0 - p.ph);
          for (int yo = r.y0; yo < r.y_end && ok;) {
            const int rn = min(p.R, r.y_end - yo);
            const int top = min(p.H - 1, yo + rn - 1 - p.ph + p.kh - 1);
            while (next_row <= top && ok) {  // one x box = up to RB window rows, each converted into its own ring slot
              const int nb = min(p.RB, top + 1 - next_row), rs = e % RX;
              ok = wait_bar(bar_xf + 8 * rs, (e / RX) & 1, status, 37, abort_flag);
              if (!ok) break;
              const float* raw = reinterpret_cast<const float*>(smem + p.off_raw_x + (uint32_t)rs * p.raw_x_bytes);
              const int off0 = (next_row * p.W + r.c0 - p.pw) & 3;  // distance of the box's first element to the 16-byte boundary below
              for (int k = 0; k < nb && ok; ++k) {
                const int bs = ring.pos;
                if (ring.wrapped) ok = wait_bar(bar_be + 8 * bs, ring.par ^ 1u, status, 38, abort_flag);
                ring.advance(p.DB);
                if (!ok) break;
                const int el = off0 + k * p.W, off = el & 3;
                const float* row = raw + (el & ~3);
                char* slot = smem + p.off_b + (uint32_t)bs * 2u * p.b_img_bytes;
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                  if (it_c4[k2] >= 0) {
                    const float* src = row + it_src[k2];
                    char* dst = slot + it_dst[k2];
                    switch (off) {
                      case 0: convert_x_item<0>(src, it_mask[k2], p.kw, dst, kx_step, p.b_img_bytes); break;
                      case 1: convert_x_item<1>(src, it_mask[k2], p.kw, dst, kx_step, p.b_img_bytes); break;
                      case 2: convert_x_item<2>(src, it_mask[k2], p.kw, dst, kx_step, p.b_img_bytes); break;
                      default: convert_x_item<3>(src, it_mask[k2], p.kw, dst, kx_step, p.b_img_bytes); break;
                    }
                  }
                }
                fence_async_smem();  // the tensor core reads these stores through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_bf + 8 * bs);
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_xe + 8 * rs);
              next_row += nb;
              ++e;
            }
            yo += rn;
          }
        } else {
          // the g row of every unit -> an A slot in tensor memory (this thread: one output channel, hi or lo part)
          constexpr int NC = P / 2;               // this warp's pixels of a row: [col0, col0 + NC)
          const int col0 = half * NC;
          const uint32_t g_mask = (r.swv >= 32 ? 0xffffffffu : ((1u << r.swv) - 1u)) >> col0;
          for (int yo = r.y0; yo < r.y_end && ok;) {
            const int rn = min(p.R, r.y_end - yo);
            for (int k0 = 0; k0 < rn && ok; k0 += p.GL, ++e) {  // one g box = the rows of up to GL units (e counts g boxes here)
              const int rs = e % RG, nu = min(p.GL, rn - k0);
              ok = wait_bar(bar_gf + 8 * rs, (e / RG) & 1, status, 39, abort_flag);
              if (!ok) break;
              const float* raw = reinterpret_cast<const float*>(smem + (uint32_t)rs * p.raw_g_bytes) + co_l * p.BWg;
              const int off0 = ((yo + k0) * p.Wo + r.c0) & 3;
              for (int k = 0; k < nu && ok; ++k, ++i) {
                const int sa = i & (p.DA - 1);
                if (i >= p.DA) ok = wait_bar(bar_ae + 8 * sa, ((i >> p.da_shift) - 1) & 1, status, 40, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const int el = off0 + k * p.Wo + col0, off = el & 3;
                const float* rr = raw + (el & ~3);
                const uint32_t taddr = tmem_base + t_lane + a_col0 + (uint32_t)(sa * P + col0);
                float sum;
                switch (off) {
                  case 0: sum = convert_g_row<NC, 0>(rr, g_mask, part, taddr); break;
                  case 1: sum = convert_g_row<NC, 1>(rr, g_mask, part, taddr); break;
                  case 2: sum = convert_g_row<NC, 2>(rr, g_mask, part, taddr); break;
                  default: sum = convert_g_row<NC, 3>(rr, g_mask, part, taddr); break;
                }
                db_acc += sum;
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_af + 8 * sa);
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_ge + 8 * rs);
            }
            yo += rn;
          }
        }
        u += r.y_end - r.y0;
      }
      if (!ok) break;
      // ---- flush this segment's accumulators as one partial: ws[partial][channel][ky * N + kx * CIT + ci] ----
      ok = __all_sync(0xffffffffu, wait_bar(bar_df, sg & 1, status, 41, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t started = *started_word;
      float* dst = p.ws + (((size_t)(combo * p.cpc + slot_id) * p.SEG + sg) * kCoTile + co_l) * (size_t)p.row_len;
      const int chunks = p.row_len / 16;   // row_len = kh * N, N a multiple of 16
      int col = cgrp * 16, ky = 0, ky_end = p.N;   // columns [ky * N, ky_end) belong to kernel row ky
      for (int cc = cgrp; cc < chunks; cc += 4, col += 64) {
        while (col >= ky_end) { ++ky; ky_end += p.N; }
        uint32_t v[16];
        if ((started >> ky) & 1u) {
          tmem_ld16_nowait(tmem_base + t_lane + (uint32_t)col, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {  // hi row (even lane) + lo row (odd lane) of the same channel
          const float mine = __uint_as_float(v[j]);
          f[j] = mine + __shfl_xor_sync(0xffffffffu, mine, 1);
        }
        if (part == 0) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(dst + col + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_de);  // the accumulators may be overwritten
    }
    // bias gradient partial: the hi lanes of the g converters hold the row sums of their channel
    if (ok && p.ws_db && cit == 0 && !x_group && part == 0 && half == 1) db_scratch[co_l] = db_acc;  // second half of the pixels
    db_half0 = ok && p.ws_db && cit == 0 && !x_group && part == 0 && half == 0;
    db_value = db_acc;
    db_channel = co_l;
  }
  tc_fence_before();
  __syncthreads();
  if (db_half0) p.ws_db[(size_t)(cot * p.cpc + slot_id) * kCoTile + db_channel] = db_value + db_scratch[db_channel];
  if (warp == kConvWarps + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dw[co, ci, ky, kx] = sum of the partials in a fixed order.  A block covers 32 consecutive elements of a partial tile
// ([64 channels][ky][kx][ci], the accumulators' own order) times 8 groups of partials: every thread adds its few
// partials, then the 8 group sums of an element are added in order and written to the element's place in dw.  The
// bias-gradient partials ([channel tile][CTA][64]) are further "elements" behind the last tile.
template <int GROUPS>
__global__ void __launch_bounds__(32 * GROUPS) conv_dw_finish_kernel(const float* __restrict__ ws, const float* __restrict__ ws_db,
                                                               float* __restrict__ dw, float* __restrict__ db, int Cout, int Cin,
                                                               int kh, int kw, int CIT, int n_cit, int NP, int cpc, int tile_elems,
                                                               int dw_elems, int db_elems) {
  __shared__ float red[GROUPS][33];
  const int lane_o = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int o = (int)blockIdx.x * 32 + lane_o;
  const float* src = nullptr;
  float* out = nullptr;
  size_t stride = 0;
  int n_part = 0;
  if (o < dw_elems) {  // element of [combo][64][kh][kw][CIT]
    const int combo = o / tile_elems, r0 = o - combo * tile_elems;
    const int row_len = kh * kw * CIT;
    const int col = r0 / row_len, r1 = r0 - col * row_len;
    const int ky = r1 / (kw * CIT), r2 = r1 - ky * kw * CIT;
    const int kx = r2 / CIT, cil = r2 - kx * CIT;
    const int cot = combo / n_cit, cit = combo - cot * n_cit;
    const int co = cot * kCoTile + col, ci = cit * CIT + cil;
    if (co < Cout && ci < Cin) out = dw + ((co * Cin + ci) * kh + ky) * kw + kx;
    src = ws + (size_t)combo * NP * tile_elems + r0;
    stride = (size_t)tile_elems;
    n_part = NP;
  } else if (o < dw_elems + db_elems) {  // bias gradient of channel co
    const int co = o - dw_elems;
    if (co < Cout) out = db + co;
    src = ws_db + (size_t)(co >> 6) * cpc * kCoTile + (co & 63);
    stride = kCoTile;
    n_part = cpc;
  }
  float acc = 0.f;
  if (out) {
    const int per = (n_part + GROUPS - 1) / GROUPS, p0 = grp * per, p1 = min(n_part, p0 + per);
    int pp = p0;
    for (; pp + 8 <= p1; pp += 8) {  // eight loads in flight per thread
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldg(src + (pp + j) * stride);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += v[j];
    }
    for (; pp < p1; ++pp) acc += __ldg(src + pp * stride);
  }
  red[grp][lane_o] = acc;
  __syncthreads();
  if (grp == 0 && out) {
    float s = red[0][lane_o];
#pragma unroll
    for (int g2 = 1; g2 < GROUPS; ++g2) s += red[g2][lane_o];
    *out = s;
  }
}

// The same sum for tiles whose innermost extent (CIT) is a multiple of four: a thread owns four consecutive elements, reads
// them with 128-bit loads and has all its partials in flight at once (the sum is a chain of dependent round trips to the L2
// otherwise: three rounds of eight loads took 7.8 us for 148 partials of 74 KB).  Threads: 32 element quads x GROUPS.
template <int GROUPS, int CHUNK>
__global__ void __launch_bounds__(32 * GROUPS) conv_dw_finish_vec_kernel(const float* __restrict__ ws, const float* __restrict__ ws_db,
                                                                   float* __restrict__ dw, float* __restrict__ db, int Cout, int Cin,
                                                                   int kh, int kw, int CIT, int n_cit, int NP, int cpc, int tile_elems,
                                                                   int dw_elems, int db_elems) {
  __shared__ float4 red[GROUPS][32];
  const int lane_o = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int o = ((int)blockIdx.x * 32 + lane_o) * 4;
  const float* src = nullptr;
  float* out = nullptr;
  int out_step = 0, n_out = 0;  // the four results go to out, out + out_step, ...; n_out of them exist
  size_t stride = 0;
  int n_part = 0;
  if (o < dw_elems) {  // four consecutive input channels of [combo][64][kh][kw][CIT]
    const int combo = o / tile_elems, r0 = o - combo * tile_elems;
    const int row_len = kh * kw * CIT;
    const int col = r0 / row_len, r1 = r0 - col * row_len;
    const int ky = r1 / (kw * CIT), r2 = r1 - ky * kw * CIT;
    const int kx = r2 / CIT, cil = r2 - kx * CIT;
    const int cot = combo / n_cit, cit = combo - cot * n_cit;
    const int co = cot * kCoTile + col, ci = cit * CIT + cil;
    if (co < Cout && ci < Cin) {
      out = dw + ((co * Cin + ci) * kh + ky) * kw + kx;
      out_step = kh * kw;
      n_out = min(4, Cin - ci);
    }
    src = ws + (size_t)combo * NP * tile_elems + r0;
    stride = (size_t)tile_elems;
    n_part = NP;
  } else if (o < dw_elems + db_elems) {  // bias gradient of channels co .. co+3
    const int co = o - dw_elems;
    if (co < Cout) {
      out = db + co;
      out_step = 1;
      n_out = min(4, Cout - co);
    }
    src = ws_db + (size_t)(co >> 6) * cpc * kCoTile + (co & 63);
    stride = kCoTile;
    n_part = cpc;
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (out) {
    const int per = (n_part + GROUPS - 1) / GROUPS, p0 = grp * per, p1 = min(n_part, p0 + per);
    for (int pp = p0; pp < p1; pp += CHUNK) {
      float4 v[CHUNK];
#pragma unroll
      for (int j = 0; j < CHUNK; ++j)
        v[j] = pp + j < p1 ? __ldg(reinterpret_cast<const float4*>(src + (size_t)(pp + j) * stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < CHUNK; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    }
  }
  red[grp][lane_o] = acc;
  __syncthreads();
  if (grp == 0 && out) {
    float4 t = red[0][lane_o];
#pragma unroll
    for (int g2 = 1; g2 < GROUPS; ++g2) {
      const float4 u = red[g2][lane_o];
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    out[0] = t.x;
    if (n_out > 1) out[out_step] = t.y;
    if (n_out > 2) out[2 * out_step] = t.z;
    if (n_out > 3) out[3 * out_step] = t.w;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
    cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 3-D map over t[Nb][C][HW] (fp32) with a box of (bw, ct, 1) elements; elements outside the tensor read as zero.
inline bool make_map(CUtensorMap* m, const float* t, int Nb, int C, int HW, int bw, int ct) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)HW, (cuuint64_t)C, (cuuint64_t)Nb};
  const cuuint64_t strides[2] = {(cuuint64_t)HW * 4, (cuuint64_t)C * HW * 4};
  const cuuint32_t box[3] = {(cuuint32_t)bw, (cuuint32_t)ct, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(t), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline int odd_quads(int floats) {  // smallest 4 * odd >= floats
  int qd = (floats + 3) / 4;
  if ((qd & 1) == 0) ++qd;
  return qd * 4;
}

}  // namespace dw
}  // namespace tc

// dw[Cy, Cx, kh, kw] (and db[Cy] when not null) for a unit-stride convolution.  Returns RT_ERR_UNIMPLEMENTED when the shape
// does not fit this kernel (the caller then takes the general path).  With db_done the caller learns whether db was written.
rt_status rt_conv_dw_tma_internal(rt_ctx* ctx, const float* x, const float* y, const ConvGeom& g, float* dw, float* db) {
  using namespace tc;
  using namespace tc::dw;
  if (g.sh != 1 || g.sw != 1 || g.kh > kMaxKh || g.kw > kMaxKw || g.kh < 1 || g.kw < 1) return RT_ERR_UNIMPLEMENTED;
  if (g.ph >= g.kh || g.pw >= g.kw || g.ph < 0 || g.pw < 0) return RT_ERR_UNIMPLEMENTED;
  if (g.Cx < 8 || g.Cy < 8 || g.Hy < 1 || g.Wy < 1 || g.Nb < 1) return RT_ERR_UNIMPLEMENTED;
  const int HWx = g.Hx * g.Wx, HWy = g.Hy * g.Wy;
  if ((HWx & 3) || (HWy & 3) || !rt_aligned16(x) || !rt_aligned16(y)) return RT_ERR_UNIMPLEMENTED;  // TMA strides / base: 16 bytes
  if ((int64_t)g.Nb * g.Cx * HWx >= (1ll << 31) || (int64_t)g.Nb * g.Cy * HWy >= (1ll << 31)) return RT_ERR_UNIMPLEMENTED;
  Params p{};
  p.Nb = g.Nb; p.Cin = g.Cx; p.Cout = g.Cy; p.H = g.Hx; p.W = g.Wx; p.Ho = g.Hy; p.Wo = g.Wy;
  p.kh = g.kh; p.kw = g.kw; p.ph = g.ph; p.pw = g.pw;
  p.nseg = (p.Wo + 31) / 32;
  p.SW = (p.Wo + p.nseg - 1) / p.nseg;
  const int P = p.SW <= 8 ? 8 : (p.SW <= 16 ? 16 : 32);
  // input channels per tile: kh accumulators of N = kw * CIT columns plus the A slots must fit the 512 tensor-memory columns
  int cit = g.Cx >= 32 ? 32 : (g.Cx + 7) / 8 * 8;
  auto n_of = [&](int c) { return g.kw * c; };
  p.R = P == 32 ? 2 : 4;
  p.DA = 2 * p.R;
  p.da_shift = p.DA == 8 ? 3 : 2;
  while (cit >= 8 && (g.kh * n_of(cit) + p.DA * P > (int)kTmemCols || n_of(cit) > 256)) cit -= 8;
  if (cit >= 16 && (n_of(cit) & 15)) cit = cit / 16 * 16;   // N must be a multiple of 16
  if (cit < 8 || (n_of(cit) & 15)) return RT_ERR_UNIMPLEMENTED;
  p.CIT = cit;
  p.N = n_of(cit);
  p.n_cot = (g.Cy + kCoTile - 1) / kCoTile;
  p.n_cit = (g.Cx + cit - 1) / cit;
  p.n_combo = p.n_cot * p.n_cit;
  if (p.n_combo > ctx->sm_count) return RT_ERR_UNIMPLEMENTED;
  const int64_t units = (int64_t)g.Nb * p.nseg * p.Ho;
  if (units >= (1ll << 30)) return RT_ERR_UNIMPLEMENTED;
  p.units = (int)units;
  p.cpc = ctx->sm_count / p.n_combo;
  if (p.cpc > p.units) p.cpc = p.units;
  // at most ~1024 accumulations per accumulator and segment: 2 MMAs per K-step
  const int per = (p.units + p.cpc - 1) / p.cpc;
  const int seg_units = max(1, 1024 / (2 * (P / 8)));
  p.SEG = (per + seg_units - 1) / seg_units;
  p.row_len = cit * g.kh * g.kw;
  p.GL = p.RB = p.nseg == 1 ? p.R : 1;
  p.BWg = odd_quads(3 + (p.GL - 1) * p.Wo + P + 4);   // what convert_g_row reads of the last row of a box
  p.BWx = odd_quads(3 + (p.RB - 1) * p.W + P + 8);    // ... and convert_x_item
  if (p.BWg > 256 || p.BWx > 256) {  // a TMA box is at most 256 elements wide
    p.GL = p.RB = 1;
    p.BWg = odd_quads(P + 4);
    p.BWx = odd_quads(P + 8);
  }
  p.raw_g_bytes = (uint32_t)(kCoTile * p.BWg * 4);
  p.raw_x_bytes = (uint32_t)(cit * p.BWx * 4);
  p.b_img_bytes = (uint32_t)(p.N * P * 4);
  p.DB = min(kMaxDB, g.kh - 1 + 2 * p.R);   // the window of one group plus the new rows of the next
  p.off_raw_x = RG * p.raw_g_bytes;
  p.off_b = p.off_raw_x + RX * p.raw_x_bytes;
  p.off_bar = (p.off_b + (uint32_t)p.DB * 2u * p.b_img_bytes + 127u) & ~127u;
  const uint32_t smem_bytes = p.off_bar + kNumBars * 8 + 16 + kCoTile * 4;
  if (smem_bytes > 227u * 1024u) return RT_ERR_UNIMPLEMENTED;
  p.d_Ho.init(p.Ho);
  p.d_nseg.init(p.nseg);

  CUtensorMap map_g, map_x;
  if (!make_map(&map_g, y, g.Nb, g.Cy, HWy, p.BWg, kCoTile) || !make_map(&map_x, x, g.Nb, g.Cx, HWx, p.BWx, cit)) return RT_ERR_UNIMPLEMENTED;

  const int NP = p.cpc * p.SEG;
  RtScratch ws(ctx), wsdb(ctx);
  rt_status st = ws.alloc(sizeof(float) * (size_t)p.n_combo * NP * kCoTile * p.row_len);
  if (st != RT_OK) return st;
  p.ws = ws.as<float>();
  if (db) {
    st = wsdb.alloc(sizeof(float) * (size_t)p.n_cot * p.cpc * kCoTile);
    if (st != RT_OK) return st;
    p.ws_db = wsdb.as<float>();
  }
  const int grid = p.n_combo * p.cpc;
  auto launch = [&](auto kern) -> rt_status {
    RT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    kern<<<grid, kThreads, smem_bytes, ctx->stream>>>(map_g, map_x, p, ctx->device_status);
    RT_LAUNCHED(ctx);
    return RT_OK;
  };
  st = P == 8 ? launch(conv_dw_kernel<8>) : (P == 16 ? launch(conv_dw_kernel<16>) : launch(conv_dw_kernel<32>));
  if (st != RT_OK) return st;
  const int tile_elems = kCoTile * p.row_len, dw_elems = p.n_combo * tile_elems, db_elems = db ? p.n_cot * kCoTile : 0;
  if (cit % 4 == 0)
    conv_dw_finish_vec_kernel<16, 12><<<((dw_elems + db_elems) / 4 + 31) / 32, 512, 0, ctx->stream>>>(
        p.ws, p.ws_db, dw, db, g.Cy, g.Cx, g.kh, g.kw, cit, p.n_cit, NP, p.cpc, tile_elems, dw_elems, db_elems);
  else
    conv_dw_finish_kernel<8><<<(dw_elems + db_elems + 31) / 32, 256, 0, ctx->stream>>>(p.ws, p.ws_db, dw, db, g.Cy, g.Cx, g.kh, g.kw, cit, p.n_cit,
                                                                                  NP, p.cpc, tile_elems, dw_elems, db_elems);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

