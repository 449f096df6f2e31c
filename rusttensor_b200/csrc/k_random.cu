// Random tensor factories on the device: uniform, normal, Bernoulli (Backend::random_uniform / random_normal /
// bernoulli, src/backend/mod.rs:61-69; kaiming_uniform, mod.rs:57, is the uniform case with bound sqrt(6 / fan_in),
// src/init.rs:26-32).
//
// The reference draws from rand's thread-local generator, which cannot be seeded, so no sequence of values exists to
// match: parity means the same distributions, ranges and error behaviour.  Here the generator is counter based
// (Philox-4x32 with 10 rounds, as published by Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): element i
// of a call is a pure function of (seed, stream offset + i / 4), so results do not depend on the launch geometry, a seed
// reproduces a run, and consecutive calls continue the stream.
#include "rt_internal.cuh"

namespace {

constexpr uint32_t kPhiloxM0 = 0xD2511F53u, kPhiloxM1 = 0xCD9E8D57u, kPhiloxW0 = 0x9E3779B9u, kPhiloxW1 = 0xBB67AE85u;

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(kPhiloxM0, ctr.x), lo0 = kPhiloxM0 * ctr.x;
    const uint32_t hi1 = __umulhi(kPhiloxM1, ctr.z), lo1 = kPhiloxM1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += kPhiloxW0;
    key.y += kPhiloxW1;
  }
  return ctr;
}

// 24 random bits -> [0, 1): every value is a multiple of 2^-24, so 1.0 is never produced
__device__ __forceinline__ float unit_float(uint32_t bits) { return (float)(bits >> 8) * (1.0f / 16777216.0f); }

enum { kUniform = 0, kNormal = 1, kBernoulli = 2 };

template <int KIND>
__global__ void __launch_bounds__(256) random_kernel(float* __restrict__ out, int64_t n, float a, float b, uint64_t seed, uint64_t offset) {
  const int64_t groups = (n + 3) / 4;
  for (int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < groups; gidx += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t c = offset + (uint64_t)gidx;
    const uint4 r = philox4x32_10(make_uint4((uint32_t)c, (uint32_t)(c >> 32), 0u, 0u), make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    float v[4];
    if (KIND == kUniform) {  // low + (high - low) * u, kept below high (rand's Uniform samples [low, high))
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float t = a + (b - a) * unit_float(w[j]);
        if (t >= b) t = nextafterf(b, a);
        v[j] = t;
      }
    } else if (KIND == kNormal) {  // Box-Muller on two pairs of uniforms; 1 - u lies in (0, 1]
      const float u0 = 1.0f - unit_float(r.x), u1 = unit_float(r.y), u2 = 1.0f - unit_float(r.z), u3 = unit_float(r.w);
      const float m0 = sqrtf(-2.0f * logf(u0)), m1 = sqrtf(-2.0f * logf(u2));
      float s0, c0, s1, c1;
      sincospif(2.0f * u1, &s0, &c0);
      sincospif(2.0f * u3, &s1, &c1);
      v[0] = a + b * (m0 * c0); v[1] = a + b * (m0 * s0); v[2] = a + b * (m1 * c1); v[3] = a + b * (m1 * s1);
    } else {  // 1.0 with probability a
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = unit_float(w[j]) < a ? 1.0f : 0.0f;
    }
    const int64_t i0 = gidx * 4;
    if (i0 + 3 < n && rt_aligned16(out)) {
      *reinterpret_cast<float4*>(out + i0) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + j < n) out[i0 + j] = v[j];
    }
  }
}

template <int KIND>
rt_status launch_random(rt_ctx* ctx, float* out, int64_t n, float a, float b, uint64_t seed, uint64_t offset) {
  if (n <= 0) return RT_OK;
  RT_CHECK_PTR(ctx, out);
  random_kernel<KIND><<<rt_grid_for(ctx, (n + 3) / 4, 256), 256, 0, ctx->stream>>>(out, n, a, b, seed, offset);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

}  // namespace

extern "C" {

rt_status rt_random_uniform(rt_ctx* ctx, float* out, int64_t n, float low, float high, uint64_t seed, uint64_t offset) {
  RT_CHECK_CTX(ctx);
  // rand's Uniform::new rejects an empty or non-finite range (Error::InitializationError in the reference)
  if (!(low < high) || !isfinite(low) || !isfinite(high) || !isfinite(high - low))
    RT_FAIL(ctx, RT_ERR_INITIALIZATION, "random_uniform: invalid range [%g, %g)", low, high);
  return launch_random<kUniform>(ctx, out, n, low, high, seed, offset);
}

rt_status rt_random_normal(rt_ctx* ctx, float* out, int64_t n, float mean, float std_dev, uint64_t seed, uint64_t offset) {
  RT_CHECK_CTX(ctx);
  if (!isfinite(std_dev)) RT_FAIL(ctx, RT_ERR_INITIALIZATION, "random_normal: standard deviation %g", std_dev);  // rand_distr: BadVariance
  return launch_random<kNormal>(ctx, out, n, mean, std_dev, seed, offset);
}

rt_status rt_bernoulli(rt_ctx* ctx, float* out, int64_t n, float p, uint64_t seed, uint64_t offset) {
  RT_CHECK_CTX(ctx);
  if (!(p >= 0.0f && p <= 1.0f)) RT_FAIL(ctx, RT_ERR_INITIALIZATION, "bernoulli: probability %g outside [0, 1]", p);
  return launch_random<kBernoulli>(ctx, out, n, p, 0.f, seed, offset);
}

}  // extern "C"
