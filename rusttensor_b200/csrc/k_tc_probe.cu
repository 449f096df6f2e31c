// Issue-rate probe for tcgen05.mma.kind::tf32: how many SM cycles one MMA of a given shape occupies
// the tensor pipe when MMAs are issued back to back.  The convolution and GEMM kernels of this
// library choose their tile shapes from these numbers (measured on a B200, K = 8: with A in shared
// memory an M = 128 MMA costs about 32 + N/4 cycles up to N = 128 and N/2 beyond, the shared-memory
// read of A being the floor; with A in tensor memory it costs N/2 for every N; M = 64 runs at half
// the rate), so the measurement ships with the library and `bench.py --mma-rate` prints it.
//
// One CTA, one warp issues `iters` MMAs (one elected lane), then one tcgen05.commit; the time from the
// first issue to the completion of the commit is divided by `iters`.  Operands are zeros in shared
// memory (K-major, no swizzle) or, for the A operand, in tensor memory.  The wait is bounded like
// every other wait in this library.
#include "rt_internal.cuh"
#include "tc_common.cuh"

namespace tc {
namespace probe {

constexpr int kThreads = 128;
constexpr uint32_t kSmemBytes = 64 * 1024;

__global__ void __launch_bounds__(kThreads, 1) issue_rate_kernel(int m, int n, int a_in_tmem, int iters, long long* out, int* status) {
  extern __shared__ __align__(1024) char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t i = threadIdx.x; i < kSmemBytes / 16; i += blockDim.x) reinterpret_cast<float4*>(smem)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fence_async_smem();
  if (warp == 0) tmem_alloc(smem_u32(&slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (warp == 0) {
    // A: rows x 32 bytes, 8-row groups 256 bytes apart (two core matrices of 128 bytes per group); B likewise.
    const uint32_t a0 = smem_u32(smem), b0 = a0 + 16 * 1024;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
    const uint64_t da = make_desc(a0, 128, 256), db = make_desc(b0, 128, 256);
    const uint32_t a_tmem = tmem + 256;  // columns 256..263 hold the A operand of the tensor-memory form
    const long long t0 = clock64();
    if (a_in_tmem) {
      for (int it = 0; it < iters; ++it)
        asm volatile(
            "{\n\t.reg .pred pe, pt;\n\t"
            "elect.sync _|pe, 0xffffffff;\n\t"
            "setp.eq.b32 pt, 0, 0;\n\t"
            "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, pt;\n\t}" ::"r"(tmem), "r"(a_tmem), "l"(db), "r"(idesc)
            : "memory");
    } else {
      for (int it = 0; it < iters; ++it)
        asm volatile(
            "{\n\t.reg .pred pe, pt;\n\t"
            "elect.sync _|pe, 0xffffffff;\n\t"
            "setp.eq.b32 pt, 0, 0;\n\t"
            "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, pt;\n\t}" ::"r"(tmem), "l"(da), "l"(db), "r"(idesc)
            : "memory");
    }
    umma_commit_elect(smem_u32(&bar));
    const long long t1 = clock64();
    mbar_wait(smem_u32(&bar), 0, status, 9);
    const long long t2 = clock64();
    if (lane == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace probe
}  // namespace tc

extern "C" rt_status rt_tc_issue_rate(rt_ctx* ctx, int m, int n, int a_in_tmem, int iters, double* issue_cycles,
                                      double* complete_cycles) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, issue_cycles);
  RT_CHECK_PTR(ctx, complete_cycles);
  // legal shapes of tcgen05.mma.cta_group::1.kind::tf32: M = 64 with N % 8 == 0, M = 128 with N % 16 == 0, 8/16 <= N <= 256
  if (!((m == 64 && n % 8 == 0 && n >= 8) || (m == 128 && n % 16 == 0 && n >= 16)) || n > 256 || iters < 1 || iters > (1 << 16))
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_tc_issue_rate: unsupported shape M=%d N=%d iters=%d", m, n, iters);
  using namespace tc::probe;
  RtScratch out(ctx);
  rt_status st = out.alloc(2 * sizeof(long long));
  if (st != RT_OK) return st;
  RT_CUDA(ctx, cudaFuncSetAttribute(issue_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  long long host[2] = {0, 0};
  for (int rep = 0; rep < 2; ++rep) {  // the second run is the measurement (instruction cache warm)
    issue_rate_kernel<<<1, kThreads, kSmemBytes, ctx->stream>>>(m, n, a_in_tmem, iters, out.as<long long>(), ctx->device_status);
    RT_LAUNCHED(ctx);
  }
  st = rt_memcpy_d2h(ctx, host, out.ptr, sizeof(host));
  if (st != RT_OK) return st;
  *issue_cycles = (double)host[0] / iters;
  *complete_cycles = (double)host[1] / iters;
  return RT_OK;
}
