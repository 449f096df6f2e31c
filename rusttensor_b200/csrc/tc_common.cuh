// PTX wrappers shared by the tensor-core (tcgen05) kernels: mbarriers with bounded waits, tensor
// memory allocation, UMMA issue / commit, accumulator loads, shared-memory matrix descriptors.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tc {

constexpr uint32_t kSpinLimit = 1u << 22;

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Records `code` in the context's status word (host memory mapped into the device's address space) unless an earlier
// code is still there.  Concurrent writers may overwrite each other: any non-zero code reports the failure.
__device__ __forceinline__ void record_status(int* status, int code) {
  volatile int* s = status;
  if (*s == 0) *s = code;
  __threadfence_system();
}
// Bounded wait.  Returns false (and records `code`) when the barrier never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  record_status(status, code);
  return false;
}
// Bulk asynchronous copy global -> shared memory of this CTA, completion counted in bytes on an mbarrier.
// Addresses and size must be multiples of 16 bytes.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Accumulator loads that do not wait: issue several, then tmem_wait_ld() once.
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (no swizzle, descriptor version 1).  For a K-major operand `lbo`
// is the byte distance between core matrices (8 rows x 16 bytes) adjacent along K and `sbo` the
// distance between 8-row groups; for an MN-major operand `sbo` is the distance between groups of
// four MN elements and `lbo` the distance between groups of eight K.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// The three MMAs of one 3xTF32 K-step in a single asm block: cross terms lo*hi and hi*lo into accumulator
// `d_cross`, hi*hi into `d_main`.  Descriptors are passed as (low word, high word); only the low word (start address)
// changes from step to step.  Called by every lane of a converged warp (so that the operands stay warp-uniform);
// one elected lane issues.
__device__ __forceinline__ void umma_tf32_step_elect(uint32_t d_cross, uint32_t d_main, uint32_t a_hi_lo32, uint32_t a_lo_lo32,
                                                     uint32_t a_hi32, uint32_t b_hi_lo32, uint32_t b_lo_lo32, uint32_t b_hi32,
                                                     uint32_t idesc, uint32_t acc_cross, uint32_t acc_main) {
  asm volatile(
      "{\n\t.reg .pred pc, pm, pt, pe;\n\t"
      ".reg .b64 dah, dal, dbh, dbl;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pc, %9, 0;\n\t"
      "setp.ne.b32 pm, %10, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 dah, {%2, %4};\n\t"
      "mov.b64 dal, {%3, %4};\n\t"
      "mov.b64 dbh, {%5, %7};\n\t"
      "mov.b64 dbl, {%6, %7};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], dal, dbh, %8, pc;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], dah, dbl, %8, pt;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%1], dah, dbh, %8, pm;\n\t}"
      ::"r"(d_cross), "r"(d_main), "r"(a_hi_lo32), "r"(a_lo_lo32), "r"(a_hi32), "r"(b_hi_lo32), "r"(b_lo_lo32), "r"(b_hi32),
        "r"(idesc), "r"(acc_cross), "r"(acc_main)
      : "memory");
}
// One 3xTF32 K-step as two MMAs: the B operand tile holds the hi rows followed by the lo rows
// (2N rows), so A_hi x [B_hi; B_lo] yields hi*hi and hi*lo side by side in `d_wide` (2N columns), and
// A_lo x B_hi goes to `d_cross` (N columns).  An MMA with N <= 128 costs the same whatever N is, so
// this is a third cheaper than three separate MMAs.  Issued by one elected lane of a converged warp.
__device__ __forceinline__ void umma_tf32_pair_elect(uint32_t d_wide, uint32_t d_cross, uint32_t a_hi_lo32, uint32_t a_lo_lo32,
                                                     uint32_t a_hi32, uint32_t b_lo32, uint32_t b_hi32, uint32_t idesc_2n,
                                                     uint32_t idesc_n, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred pa, pe;\n\t"
      ".reg .b64 dah, dal, db;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %9, 0;\n\t"
      "mov.b64 dah, {%2, %4};\n\t"
      "mov.b64 dal, {%3, %4};\n\t"
      "mov.b64 db, {%5, %6};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%0], dah, db, %7, pa;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::tf32 [%1], dal, db, %8, pa;\n\t}"
      ::"r"(d_wide), "r"(d_cross), "r"(a_hi_lo32), "r"(a_lo_lo32), "r"(a_hi32), "r"(b_lo32), "r"(b_hi32), "r"(idesc_2n),
        "r"(idesc_n), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred pe;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
      : "memory");
}
// Low / high words of the shared-memory matrix descriptor of make_desc.
__device__ __forceinline__ uint32_t desc_lo32(uint32_t saddr, uint32_t lbo) { return ((saddr >> 4) & 0x3FFF) | ((lbo >> 4) << 16); }
__device__ __forceinline__ uint32_t desc_hi32(uint32_t sbo) { return ((sbo >> 4) & 0x3FFF) | (1u << 14); }
// Instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// a = hi + lo with hi = a with the low 13 mantissa bits cleared (exactly representable in TF32)
__device__ __forceinline__ void split4(const float (&v)[4], float4& hi, float4& lo) {
  float h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __uint_as_float(__float_as_uint(v[i]) & 0xFFFFE000u);
  hi = make_float4(h[0], h[1], h[2], h[3]);
  lo = make_float4(v[0] - h[0], v[1] - h[1], v[2] - h[2], v[3] - h[3]);
}

}  // namespace tc
