// Fused optimizer steps: SGD, momentum SGD, AdaGrad and Adam, each a single pass over
// parameter, gradient and state (12 / 20 / 20 / 28 bytes of HBM traffic per parameter).
//
// The per-tensor entry points mirror the reference trait methods; rt_optimizer_step_multi
// updates a whole model (a list of tensors) in one launch, optionally clamping and scaling
// the gradient on the fly (gradient clipping and the 1/world of a data-parallel mean),
// and rt_pack_flat gathers the gradients into one flat buffer for a single all-reduce.
//
// Update formulas are written in the algebraic form of the reference CPU backend
// (src/backend/cpu.rs:32-126, 244-318).  Adam's bias corrections 1 - beta^t are computed
// once on the host with the repeated-squaring integer power the reference uses
// (f32::powi), not per thread.
#include <cmath>

#include "rt_internal.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxTensors = 48;
constexpr int kChunkLarge = kThreads * 16;  // elements per block for large models
constexpr int kChunkSmall = kThreads * 4;   // ... and when the whole model would not fill the machine otherwise

// Elements per block: one 128-bit access per thread while the model is small (every load of the step in flight at
// once: a 0.4 M-parameter model is latency-bound, not bandwidth-bound), sixteen elements per thread beyond that.
inline int chunk_for(rt_ctx* ctx, const int64_t* sizes, int n_tensors) {
  int64_t total = 0;
  for (int i = 0; i < n_tensors; ++i) total += sizes[i] > 0 ? sizes[i] : 0;
  return total <= (int64_t)ctx->sm_count * 8 * kChunkLarge ? kChunkSmall : kChunkLarge;
}

struct OptArgs {
  float* p[kMaxTensors];
  const float* g[kMaxTensors];
  float* s1[kMaxTensors];
  float* s2[kMaxTensors];
  int64_t n[kMaxTensors];
  int block_start[kMaxTensors + 1];  // first block of each tensor
  int count;
  int chunk;  // elements per block
  float lr, beta1, beta2, eps, momentum, bc1, bc2, grad_scale, clip_lo, clip_hi;
  int clip;
  // Step state in device memory (rt_dp_step_begin), or null: with it the optimizer step count t is read on the device, so
  // that the launch can be replayed from a CUDA graph; need_ready makes the update conditional on the peers' gradients
  // being complete for this step (rt_dp_wait_peers).
  const int* ctrl;
  int need_ready;
};

// Words of the step state.
enum { kCtrlStep = 0, kCtrlReady = 1, kCtrlT = 2, kCtrlWaited = 3, kCtrlWords = 4 };

// compiler-rt __powisf2, the lowering of f32::powi used by the reference (cpu.rs:302-303)
__host__ __device__ inline float powi_f32(float a, int b) {
  const bool recip = b < 0;
  float r = 1.f;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.f / r : r;
}

// Per-block prologue of the optimizer kernels: Adam's bias corrections (from the host, or from the device-side step
// count) and whether the block may update at all.  Every block takes the same decision: it reads the same words.
template <int KIND>
__device__ __forceinline__ bool optimizer_prologue(const OptArgs& a, float& bc1, float& bc2) {
  __shared__ float s_bc[2];
  __shared__ int s_go;
  if (threadIdx.x == 0) {
    float b1 = a.bc1, b2 = a.bc2;
    int go = 1;
    if (a.ctrl) {
      if (KIND == 1) {
        const int t = a.ctrl[kCtrlT];
        b1 = 1.0f - powi_f32(a.beta1, t);
        b2 = 1.0f - powi_f32(a.beta2, t);
      }
      if (a.need_ready) go = a.ctrl[kCtrlReady] == a.ctrl[kCtrlStep];
    }
    s_bc[0] = b1;
    s_bc[1] = b2;
    s_go = go;
  }
  __syncthreads();
  bc1 = s_bc[0];
  bc2 = s_bc[1];
  return s_go != 0;
}

template <int KIND>
__device__ __forceinline__ void update(float& p, float g, float& s1, float& s2, const OptArgs& a, float bc1, float bc2) {
  if (a.clip) g = fminf(fmaxf(g, a.clip_lo), a.clip_hi);
  g *= a.grad_scale;
  if (KIND == 0) {  // sgd: w -= lr * dw
    p -= a.lr * g;
  } else if (KIND == 1) {  // adam
    s1 = a.beta1 * s1 + (1.0f - a.beta1) * g;
    s2 = a.beta2 * s2 + (1.0f - a.beta2) * (g * g);
    float mh = s1 / bc1, vh = s2 / bc2;
    p -= a.lr * mh / (sqrtf(vh) + a.eps);
  } else if (KIND == 2) {  // momentum: v = mu*v + g ; p -= lr*v
    s1 = a.momentum * s1 + g;
    p -= a.lr * s1;
  } else {  // adagrad: acc += g*g ; p -= lr*g/(sqrt(acc)+eps)
    s1 += g * g;
    p -= a.lr * g / (sqrtf(s1) + a.eps);
  }
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) optimizer_kernel(const __grid_constant__ OptArgs a) {
  float bc1, bc2;
  if (!optimizer_prologue<KIND>(a, bc1, bc2)) return;
  // locate the tensor this block works on
  int ti = 0;
  while (ti + 1 < a.count && (int)blockIdx.x >= a.block_start[ti + 1]) ++ti;
  int64_t base = (int64_t)(blockIdx.x - a.block_start[ti]) * a.chunk;
  int64_t n = a.n[ti];
  int64_t end = base + a.chunk < n ? base + a.chunk : n;
  float* p = a.p[ti];
  const float* g = a.g[ti];
  float* s1 = a.s1[ti];
  float* s2 = a.s2[ti];
  bool vec = rt_aligned16(p) && rt_aligned16(g) && (KIND == 0 || rt_aligned16(s1)) && (KIND != 1 || rt_aligned16(s2));
  if (vec) {
    int64_t end4 = base + ((end - base) & ~int64_t(3));
    for (int64_t i = base + threadIdx.x * 4; i < end4; i += kThreads * 4) {
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 gv = __ldg(reinterpret_cast<const float4*>(g + i));
      float4 m = make_float4(0, 0, 0, 0), v = make_float4(0, 0, 0, 0);
      if (KIND != 0) m = *reinterpret_cast<float4*>(s1 + i);
      if (KIND == 1) v = *reinterpret_cast<float4*>(s2 + i);
      update<KIND>(pv.x, gv.x, m.x, v.x, a, bc1, bc2);
      update<KIND>(pv.y, gv.y, m.y, v.y, a, bc1, bc2);
      update<KIND>(pv.z, gv.z, m.z, v.z, a, bc1, bc2);
      update<KIND>(pv.w, gv.w, m.w, v.w, a, bc1, bc2);
      *reinterpret_cast<float4*>(p + i) = pv;
      if (KIND != 0) *reinterpret_cast<float4*>(s1 + i) = m;
      if (KIND == 1) *reinterpret_cast<float4*>(s2 + i) = v;
    }
    base = end4;
  }
  for (int64_t i = base + threadIdx.x; i < end; i += kThreads) {
    float pv = p[i], m = KIND != 0 ? s1[i] : 0.f, v = KIND == 1 ? s2[i] : 0.f;
    update<KIND>(pv, g[i], m, v, a, bc1, bc2);
    p[i] = pv;
    if (KIND != 0) s1[i] = m;
    if (KIND == 1) s2[i] = v;
  }
}

// ---- optimizer step with the gradient exchange fused in (peer memory) -----------------------------------------------
constexpr int kMaxPeers = RT_DP_MAX_PEERS;
struct PeerArgs {
  const float* flat[2][kMaxPeers];  // flat[b][r] = rank r's packed gradients, buffer b (this rank's own at [b][rank])
  int world, rank;
};

__device__ __forceinline__ float4 ld_peer4(const float* p) {  // system-scope load: never served from a stale L1 line
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer1(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Same work split as optimizer_kernel; the gradient of an element is the sum, in rank order, of that element of every
// rank's flat buffer of this step (buffer = step & 1).  Runs only when rt_dp_wait_peers has marked this step ready.
template <int KIND>
__global__ void __launch_bounds__(kThreads) optimizer_peer_kernel(const __grid_constant__ OptArgs a, const __grid_constant__ PeerArgs pa) {
  float bc1, bc2;
  if (!optimizer_prologue<KIND>(a, bc1, bc2)) return;
  const int buf = a.ctrl[kCtrlStep] & 1;
  int ti = 0;
  while (ti + 1 < a.count && (int)blockIdx.x >= a.block_start[ti + 1]) ++ti;
  int64_t base = (int64_t)(blockIdx.x - a.block_start[ti]) * a.chunk;
  const int64_t n = a.n[ti];
  const int64_t end = base + a.chunk < n ? base + a.chunk : n;
  float* p = a.p[ti];
  float* s1 = a.s1[ti];
  float* s2 = a.s2[ti];
  const int64_t goff = a.g[ti] - pa.flat[0][pa.rank];  // offset of this tensor inside every flat buffer
  const bool vec = rt_aligned16(p) && ((goff & 3) == 0) && (KIND == 0 || rt_aligned16(s1)) && (KIND != 1 || rt_aligned16(s2));
  if (vec) {
    const int64_t end4 = base + ((end - base) & ~int64_t(3));
    for (int64_t i = base + threadIdx.x * 4; i < end4; i += kThreads * 4) {
      // every rank's load is issued before the first one is used (a remote load takes a few microseconds); the sum
      // then runs in rank order, the same on every rank
      float4 t[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < pa.world) t[r] = ld_peer4(pa.flat[buf][r] + goff + i);
      float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < pa.world) {
          gv.x += t[r].x; gv.y += t[r].y; gv.z += t[r].z; gv.w += t[r].w;
        }
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 m = make_float4(0, 0, 0, 0), v = make_float4(0, 0, 0, 0);
      if (KIND != 0) m = *reinterpret_cast<float4*>(s1 + i);
      if (KIND == 1) v = *reinterpret_cast<float4*>(s2 + i);
      update<KIND>(pv.x, gv.x, m.x, v.x, a, bc1, bc2);
      update<KIND>(pv.y, gv.y, m.y, v.y, a, bc1, bc2);
      update<KIND>(pv.z, gv.z, m.z, v.z, a, bc1, bc2);
      update<KIND>(pv.w, gv.w, m.w, v.w, a, bc1, bc2);
      *reinterpret_cast<float4*>(p + i) = pv;
      if (KIND != 0) *reinterpret_cast<float4*>(s1 + i) = m;
      if (KIND == 1) *reinterpret_cast<float4*>(s2 + i) = v;
    }
    base = end4;
  }
  for (int64_t i = base + threadIdx.x; i < end; i += kThreads) {
    float t[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < pa.world) t[r] = ld_peer1(pa.flat[buf][r] + goff + i);
    float g = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < pa.world) g += t[r];
    float pv = p[i], m = KIND != 0 ? s1[i] : 0.f, v = KIND == 1 ? s2[i] : 0.f;
    update<KIND>(pv, g, m, v, a, bc1, bc2);
    p[i] = pv;
    if (KIND != 0) s1[i] = m;
    if (KIND == 1) s2[i] = v;
  }
}

// Starts a step: the exchange step number and the optimizer step count advance on the device.
__global__ void dp_step_begin_kernel(int* ctrl) {
  if (threadIdx.x == 0) {
    ctrl[kCtrlStep] += 1;
    ctrl[kCtrlT] += 1;
  }
}

struct SignalArgs {
  int* flags[kMaxPeers];
  int world, rank;
};
// Runs after the pack kernel on the same stream: the packed gradients are complete in this GPU's memory when the
// peers see the flag.
__global__ void dp_signal_kernel(const SignalArgs sa, const int* ctrl) {
  const int r = threadIdx.x;
  if (r < sa.world && r != sa.rank) {
    const int step = ctrl[kCtrlStep];
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(sa.flags[r] + sa.rank), "r"(step) : "memory");
  }
}

// One block: thread r waits (bounded) until rank r has signalled this step, then the block marks the step ready - or,
// when a wait ran out, records a code in the status word and marks the step failed, so that the optimizer kernel that
// follows leaves parameters and state untouched in ALL of its blocks.
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void dp_wait_kernel(const int* flags, int world, int rank, int* ctrl, uint32_t spin_limit, int* status) {
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  const int step = ctrl[kCtrlStep];
  const int r = threadIdx.x;
  const unsigned long long t0 = global_timer_ns();
  if (r < world && r != rank) {
    const volatile int* f = flags + r;
    uint32_t spins = 0;
    while (*f < step) {
      if (++spins > spin_limit) {
        atomicMax(&bad, 16 + r);
        break;
      }
      if (spins > 32) __nanosleep(128);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // how long this rank waited for its slowest peer, accumulated in units of 64 ns (a diagnostic: read with rt_memcpy_d2h)
    ctrl[kCtrlWaited] += (int)((global_timer_ns() - t0) >> 6);
    __threadfence_system();
    if (bad) {
      volatile int* s = status;
      if (*s == 0) *s = bad;
      ctrl[kCtrlReady] = -step;
    } else {
      ctrl[kCtrlReady] = step;
    }
  }
}

struct PackArgs {
  const float* src[kMaxTensors];
  int64_t n[kMaxTensors];
  int64_t dst_off[kMaxTensors];
  int block_start[kMaxTensors + 1];
  int count;
  int chunk;  // elements per block
  float clip_lo, clip_hi;
  int clip;
};

// flat1 / ctrl may be null; with them the destination alternates with the step number (buffer = step & 1).
// SIGNAL: the block that finishes last (a ticket) also writes the step number into this rank's slot of every peer's flag
// array, which saves the separate signalling launch.  Every block makes its part of the buffer visible system-wide before it
// draws its ticket, so the buffer is complete in this GPU's memory when a peer sees the flag.
template <bool SIGNAL>
__global__ void __launch_bounds__(kThreads) pack_kernel(const __grid_constant__ PackArgs a, float* flat0, float* flat1, const int* ctrl,
                                                         const SignalArgs sa, unsigned* ticket) {
  float* __restrict__ flat = (ctrl && (ctrl[kCtrlStep] & 1)) ? flat1 : flat0;
  int ti = 0;
  while (ti + 1 < a.count && (int)blockIdx.x >= a.block_start[ti + 1]) ++ti;
  int64_t base = (int64_t)(blockIdx.x - a.block_start[ti]) * a.chunk;
  int64_t n = a.n[ti];
  int64_t end = base + a.chunk < n ? base + a.chunk : n;
  const float* s = a.src[ti];
  float* d = flat + a.dst_off[ti];
  if (rt_aligned16(s) && rt_aligned16(d)) {  // chunk and dst_off are multiples of 4 elements
    int64_t end4 = base + ((end - base) & ~int64_t(3));
    for (int64_t i = base + threadIdx.x * 4; i < end4; i += kThreads * 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(s + i));
      if (a.clip) {
        v.x = fminf(fmaxf(v.x, a.clip_lo), a.clip_hi); v.y = fminf(fmaxf(v.y, a.clip_lo), a.clip_hi);
        v.z = fminf(fmaxf(v.z, a.clip_lo), a.clip_hi); v.w = fminf(fmaxf(v.w, a.clip_lo), a.clip_hi);
      }
      *reinterpret_cast<float4*>(d + i) = v;
    }
    base = end4;
  }
  for (int64_t i = base + threadIdx.x; i < end; i += kThreads) {
    float v = s[i];
    if (a.clip) v = fminf(fmaxf(v, a.clip_lo), a.clip_hi);
    d[i] = v;
  }
  if (SIGNAL) {
    __shared__ int is_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
      if (is_last) *ticket = 0;
    }
    __syncthreads();
    const int r = threadIdx.x;
    if (is_last && r < sa.world && r != sa.rank) {
      const int step = ctrl[kCtrlStep];
      __threadfence_system();
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(sa.flags[r] + sa.rank), "r"(step) : "memory");
    }
  }
}

rt_status launch_multi(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                       float* const* s1, float* const* s2, const int64_t* sizes, float lr, float beta1, float beta2,
                       float eps, float momentum, int64_t t, float grad_scale, int clip, float clip_lo, float clip_hi,
                       const int* ctrl = nullptr) {
  if (kind < 0 || kind > 3) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "optimizer kind %d", kind);
  if (kind == 1 && t <= 0 && !ctrl) RT_FAIL(ctx, RT_ERR_INTERNAL, "Adam step called with t=0");
  const int chunk = chunk_for(ctx, sizes, n_tensors);
  for (int first = 0; first < n_tensors; first += kMaxTensors) {
    OptArgs a;
    a.count = 0;
    a.chunk = chunk;
    int blocks = 0;
    for (int i = first; i < n_tensors && a.count < kMaxTensors; ++i) {
      if (sizes[i] <= 0) continue;
      if (!params[i] || !grads[i] || (kind != 0 && !s1[i]) || (kind == 1 && !s2[i]))
        RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "optimizer step: null pointer for tensor %d", i);
      int c = a.count++;
      a.p[c] = params[i];
      a.g[c] = grads[i];
      a.s1[c] = kind != 0 ? s1[i] : nullptr;
      a.s2[c] = kind == 1 ? s2[i] : nullptr;
      a.n[c] = sizes[i];
      a.block_start[c] = blocks;
      blocks += (int)((sizes[i] + chunk - 1) / chunk);
    }
    if (a.count == 0) continue;
    a.block_start[a.count] = blocks;
    a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.momentum = momentum;
    a.grad_scale = grad_scale; a.clip = clip; a.clip_lo = clip_lo; a.clip_hi = clip_hi;
    a.bc1 = a.bc2 = 1.f;
    a.ctrl = ctrl;
    a.need_ready = 0;
    if (kind == 1 && !ctrl) {
      a.bc1 = 1.0f - powi_f32(beta1, (int)t);
      a.bc2 = 1.0f - powi_f32(beta2, (int)t);
    }
    switch (kind) {
      case 0: optimizer_kernel<0><<<blocks, kThreads, 0, ctx->stream>>>(a); break;
      case 1: optimizer_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(a); break;
      case 2: optimizer_kernel<2><<<blocks, kThreads, 0, ctx->stream>>>(a); break;
      default: optimizer_kernel<3><<<blocks, kThreads, 0, ctx->stream>>>(a); break;
    }
    RT_LAUNCHED(ctx);
  }
  return RT_OK;
}

}  // namespace

extern "C" {

rt_status rt_optimizer_step_multi(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                                  float* const* state1, float* const* state2, const int64_t* sizes, float lr, float beta1,
                                  float beta2, float epsilon, float momentum, int64_t t, float grad_scale, int clip,
                                  float clip_lo, float clip_hi) {
  RT_CHECK_CTX(ctx);
  if (n_tensors <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, params);
  RT_CHECK_PTR(ctx, grads);
  RT_CHECK_PTR(ctx, sizes);
  return launch_multi(ctx, kind, n_tensors, params, grads, state1, state2, sizes, lr, beta1, beta2, epsilon, momentum, t,
                      grad_scale, clip, clip_lo, clip_hi);
}

rt_status rt_sgd_step(rt_ctx* ctx, float* param, const float* grad, int64_t n, float lr) {
  RT_CHECK_CTX(ctx);
  return launch_multi(ctx, 0, 1, &param, &grad, nullptr, nullptr, &n, lr, 0, 0, 0, 0, 1, 1.f, 0, 0, 0);
}

rt_status rt_momentum_sgd_step(rt_ctx* ctx, float* param, const float* grad, float* velocity, int64_t n, float lr,
                               float momentum) {
  RT_CHECK_CTX(ctx);
  return launch_multi(ctx, 2, 1, &param, &grad, &velocity, nullptr, &n, lr, 0, 0, 0, momentum, 1, 1.f, 0, 0, 0);
}

rt_status rt_adagrad_step(rt_ctx* ctx, float* param, const float* grad, float* accum, int64_t n, float lr, float epsilon) {
  RT_CHECK_CTX(ctx);
  return launch_multi(ctx, 3, 1, &param, &grad, &accum, nullptr, &n, lr, 0, 0, epsilon, 0, 1, 1.f, 0, 0, 0);
}

rt_status rt_adam_step(rt_ctx* ctx, float* param, const float* grad, float* m, float* v, int64_t n, float lr, float beta1,
                       float beta2, float epsilon, int64_t t) {
  RT_CHECK_CTX(ctx);
  return launch_multi(ctx, 1, 1, &param, &grad, &m, &v, &n, lr, beta1, beta2, epsilon, 0, t, 1.f, 0, 0, 0);
}

static rt_status pack_flat_impl(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat0, float* flat1,
                                const int* ctrl, int clip, float clip_lo, float clip_hi, const SignalArgs* signal = nullptr) {
  if (n_tensors <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, srcs);
  RT_CHECK_PTR(ctx, sizes);
  RT_CHECK_PTR(ctx, flat0);
  int64_t off = 0;
  const int chunk = chunk_for(ctx, sizes, n_tensors);
  for (int first = 0; first < n_tensors; first += kMaxTensors) {
    PackArgs a;
    a.count = 0;
    a.chunk = chunk;
    int blocks = 0;
    for (int i = first; i < n_tensors && i < first + kMaxTensors; ++i) {
      int64_t padded = (sizes[i] + 3) & ~int64_t(3);  // every tensor starts on a 16-byte boundary
      if (sizes[i] > 0) {
        if (!srcs[i]) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_pack_flat: null source %d", i);
        int c = a.count++;
        a.src[c] = srcs[i];
        a.n[c] = sizes[i];
        a.dst_off[c] = off;
        a.block_start[c] = blocks;
        blocks += (int)((sizes[i] + chunk - 1) / chunk);
      }
      off += padded;
    }
    if (a.count == 0) continue;
    a.block_start[a.count] = blocks;
    a.clip = clip; a.clip_lo = clip_lo; a.clip_hi = clip_hi;
    if (signal) {
      unsigned* ticket = ctx->reduce_counters + 2 * kReduceCounterSlots + (ctx->on_side ? kAuxCounterSlots : 0) + kAuxCounterSlots - 1;
      pack_kernel<true><<<blocks, kThreads, 0, ctx->stream>>>(a, flat0, flat1, ctrl, *signal, ticket);
    } else {
      pack_kernel<false><<<blocks, kThreads, 0, ctx->stream>>>(a, flat0, flat1, ctrl, SignalArgs{}, nullptr);
    }
    RT_LAUNCHED(ctx);
  }
  return RT_OK;
}

rt_status rt_pack_flat(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat, int clip,
                       float clip_lo, float clip_hi) {
  RT_CHECK_CTX(ctx);
  return pack_flat_impl(ctx, n_tensors, srcs, sizes, flat, nullptr, nullptr, clip, clip_lo, clip_hi);
}

rt_status rt_pack_flat_alternating(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat0,
                                   float* flat1, const int* step_state, int clip, float clip_lo, float clip_hi) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, flat1);
  RT_CHECK_PTR(ctx, step_state);
  return pack_flat_impl(ctx, n_tensors, srcs, sizes, flat0, flat1, step_state, clip, clip_lo, clip_hi);
}

rt_status rt_pack_flat_signal(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat0, float* flat1,
                              const int* step_state, int clip, float clip_lo, float clip_hi, int* const* peer_flags, int rank,
                              int world) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, flat1);
  RT_CHECK_PTR(ctx, step_state);
  RT_CHECK_PTR(ctx, peer_flags);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_pack_flat_signal: rank %d of %d (at most %d peers)", rank, world, kMaxPeers);
  int live = 0;
  for (int i = 0; i < n_tensors; ++i) live += sizes && sizes[i] > 0;
  if (n_tensors > kMaxTensors || live == 0 || !ctx->reduce_counters) {  // several pack launches, or nothing to pack: signal separately
    rt_status st = pack_flat_impl(ctx, n_tensors, srcs, sizes, flat0, flat1, step_state, clip, clip_lo, clip_hi);
    return st != RT_OK ? st : rt_dp_signal_peers(ctx, peer_flags, rank, world, step_state);
  }
  SignalArgs sa;
  for (int r = 0; r < kMaxPeers; ++r) sa.flags[r] = r < world ? peer_flags[r] : nullptr;
  for (int r = 0; r < world; ++r)
    if (r != rank && !sa.flags[r]) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_pack_flat_signal: no flag array for rank %d", r);
  sa.world = world; sa.rank = rank;
  return pack_flat_impl(ctx, n_tensors, srcs, sizes, flat0, flat1, step_state, clip, clip_lo, clip_hi, &sa);
}

rt_status rt_dp_step_begin(rt_ctx* ctx, int* step_state) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, step_state);
  dp_step_begin_kernel<<<1, 32, 0, ctx->stream>>>(step_state);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_optimizer_step_multi_device_t(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                                           float* const* state1, float* const* state2, const int64_t* sizes, float lr, float beta1,
                                           float beta2, float epsilon, float momentum, const int* step_state, float grad_scale,
                                           int clip, float clip_lo, float clip_hi) {
  RT_CHECK_CTX(ctx);
  if (n_tensors <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, params);
  RT_CHECK_PTR(ctx, grads);
  RT_CHECK_PTR(ctx, sizes);
  RT_CHECK_PTR(ctx, step_state);
  return launch_multi(ctx, kind, n_tensors, params, grads, state1, state2, sizes, lr, beta1, beta2, epsilon, momentum, 0, grad_scale,
                      clip, clip_lo, clip_hi, step_state);
}

rt_status rt_dp_signal_peers(rt_ctx* ctx, int* const* peer_flags, int rank, int world, const int* step_state) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, peer_flags);
  RT_CHECK_PTR(ctx, step_state);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_dp_signal_peers: rank %d of %d (at most %d peers)", rank, world, kMaxPeers);
  SignalArgs sa;
  for (int r = 0; r < kMaxPeers; ++r) sa.flags[r] = r < world ? peer_flags[r] : nullptr;
  for (int r = 0; r < world; ++r)
    if (r != rank && !sa.flags[r]) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_dp_signal_peers: no flag array for rank %d", r);
  sa.world = world; sa.rank = rank;
  dp_signal_kernel<<<1, 32, 0, ctx->stream>>>(sa, step_state);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_dp_wait_peers(rt_ctx* ctx, const int* local_flags, int rank, int world, int* step_state, uint32_t spin_limit) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, local_flags);
  RT_CHECK_PTR(ctx, step_state);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_dp_wait_peers: rank %d of %d (at most %d peers)", rank, world, kMaxPeers);
  if (spin_limit == 0) spin_limit = 1u << 26;  // about ten seconds of polling with the back-off of the kernel
  dp_wait_kernel<<<1, 32, 0, ctx->stream>>>(local_flags, world, rank, step_state, spin_limit, ctx->device_status);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_optimizer_step_multi_peers(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                                        float* const* state1, float* const* state2, const int64_t* sizes, float lr, float beta1,
                                        float beta2, float epsilon, float momentum, float grad_scale, const float* const* flats0,
                                        const float* const* flats1, int rank, int world, const int* step_state) {
  RT_CHECK_CTX(ctx);
  if (n_tensors <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, params);
  RT_CHECK_PTR(ctx, grads);
  RT_CHECK_PTR(ctx, sizes);
  RT_CHECK_PTR(ctx, flats0);
  RT_CHECK_PTR(ctx, flats1);
  RT_CHECK_PTR(ctx, step_state);
  if (kind < 0 || kind > 3) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "optimizer kind %d", kind);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_optimizer_step_multi_peers: rank %d of %d (at most %d peers)", rank, world, kMaxPeers);
  if (n_tensors > kMaxTensors) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_optimizer_step_multi_peers: at most %d tensors", kMaxTensors);
  PeerArgs pa;
  for (int r = 0; r < kMaxPeers; ++r) {
    pa.flat[0][r] = r < world ? flats0[r] : nullptr;
    pa.flat[1][r] = r < world ? flats1[r] : nullptr;
  }
  for (int r = 0; r < world; ++r)
    if (!pa.flat[0][r] || !pa.flat[1][r]) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_optimizer_step_multi_peers: no flat buffer for rank %d", r);
  pa.world = world; pa.rank = rank;
  const int chunk = chunk_for(ctx, sizes, n_tensors);
  OptArgs a;
  a.count = 0;
  a.chunk = chunk;
  int blocks = 0;
  for (int i = 0; i < n_tensors; ++i) {
    if (sizes[i] <= 0) continue;
    if (!params[i] || !grads[i] || (kind != 0 && !state1[i]) || (kind == 1 && !state2[i]))
      RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "optimizer step: null pointer for tensor %d", i);
    int c = a.count++;
    a.p[c] = params[i];
    a.g[c] = grads[i];
    a.s1[c] = kind != 0 ? state1[i] : nullptr;
    a.s2[c] = kind == 1 ? state2[i] : nullptr;
    a.n[c] = sizes[i];
    a.block_start[c] = blocks;
    blocks += (int)((sizes[i] + chunk - 1) / chunk);
  }
  if (a.count == 0) return RT_OK;
  a.block_start[a.count] = blocks;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = epsilon; a.momentum = momentum;
  a.grad_scale = grad_scale; a.clip = 0; a.clip_lo = 0.f; a.clip_hi = 0.f;
  a.bc1 = a.bc2 = 1.f;
  a.ctrl = step_state;
  a.need_ready = 1;
  switch (kind) {
    case 0: optimizer_peer_kernel<0><<<blocks, kThreads, 0, ctx->stream>>>(a, pa); break;
    case 1: optimizer_peer_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(a, pa); break;
    case 2: optimizer_peer_kernel<2><<<blocks, kThreads, 0, ctx->stream>>>(a, pa); break;
    default: optimizer_peer_kernel<3><<<blocks, kThreads, 0, ctx->stream>>>(a, pa); break;
  }
  RT_LAUNCHED(ctx);
  return RT_OK;
}

}  // extern "C"
