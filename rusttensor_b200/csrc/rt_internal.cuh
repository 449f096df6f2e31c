// Internal declarations shared by the kernel translation units of librt_b200.so.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "../../include/rt_b200.h"

struct rt_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  // Blocks that were released while the graph was being captured.  The graph's kernels
  // still write them on every replay, so they stay out of the pool until the graph is
  // destroyed.
  std::vector<std::pair<size_t, void*>> retired;
};

struct rt_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  std::string last_error;
  // Caching allocator: freed blocks are kept per rounded size and handed out again.
  // All work is ordered on one stream, so reuse needs no extra synchronisation.
  std::multimap<size_t, void*> free_blocks;
  std::map<void*, size_t> live_blocks;
  int64_t bytes_reserved = 0, bytes_in_use = 0, n_device_allocs = 0;
  int64_t launches = 0;
  bool capturing = false;
  std::multimap<size_t, void*> capture_free;  // released during capture: reusable only inside it
  cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
  // side stream (rt_side_stream_*): `stream` points at it between begin and end
  cudaStream_t side_stream = nullptr, main_stream = nullptr;
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  bool on_side = false, side_pending = false;
  // Sections opened by the library itself (RtFork) may allocate: what they free is parked until the join, so that
  // nothing queued on the main stream in between can be handed a block the side stream still uses.
  bool side_internal = false;
  std::vector<std::pair<size_t, void*>> side_deferred;
  bool concurrent_backward = true;  // independent halves of one backward call on two streams (RT_B200_SERIAL_BACKWARD=1: off)
  // Error word written by kernels whose bounded waits expire (0 = none): one int of pinned host memory mapped into the
  // device's address space.  device_status is what kernels get, host_status the same word as the host reads it.
  int* device_status = nullptr;
  volatile int* host_status = nullptr;
  // Tickets of the kernels that finish a split sum in their last block (k_reduce.cu, k_conv_thin.cu): zero between launches.
  // 2 x kReduceCounterSlots for the column reductions, then 2 x kAuxCounterSlots; of each pair one half serves work queued on
  // the main stream and one the side stream, which may run such a kernel at the same time.
  unsigned* reduce_counters = nullptr;
  // Route large contractions to the tcgen05 3xTF32 kernels (k_gemm_tc.cu).
  bool use_tensor_cores = true;
  // Unit-stride convolution weight gradients through the TMA-fed kernel with the pixels as the reduction index
  // (k_conv_dw_tc.cu); RT_B200_CONV_DW_TMA=0 keeps the general implicit-GEMM kernel.
  bool use_tma_weight_grad = true;
  // NCCL (loaded at run time on first use)
  void* nccl_comm = nullptr;
  bool nccl_nonblocking = false;  // the communicator was created in NCCL's non-blocking mode: calls may answer "in progress"
  int64_t dp_timeout_ms = 120000; // host deadline of every wait on the communicator
  int dp_rank = 0, dp_world = 1;
};

constexpr int kReduceCounterSlots = 4096;  // per stream half: tickets of the column reductions
constexpr int kAuxCounterSlots = 128;      // per stream half, behind them: tickets of other kernels that hand partial sums over

#define RT_FAIL(ctx, code, ...)                         \
  do {                                                  \
    char _buf[512];                                     \
    snprintf(_buf, sizeof(_buf), __VA_ARGS__);          \
    if (ctx) (ctx)->last_error = _buf;                  \
    return (code);                                      \
  } while (0)

#define RT_CUDA(ctx, expr)                                                                     \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      RT_FAIL(ctx, _e == cudaErrorMemoryAllocation ? RT_ERR_OOM : RT_ERR_CUDA, "%s failed: %s", #expr, \
              cudaGetErrorString(_e));                                                         \
  } while (0)

#define RT_CHECK_CTX(ctx) \
  do {                    \
    if (!(ctx)) return RT_ERR_INVALID_OPERATION; \
  } while (0)

#define RT_CHECK_PTR(ctx, p)                                                   \
  do {                                                                         \
    if (!(p)) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "%s: null pointer %s", __func__, #p); \
  } while (0)

// Records a kernel launch and converts a launch error into a status.
#define RT_LAUNCHED(ctx)                                                                   \
  do {                                                                                     \
    (ctx)->launches++;                                                                     \
    cudaError_t _e = cudaPeekAtLastError();                                                \
    if (_e != cudaSuccess) {                                                               \
      cudaGetLastError();                                                                  \
      RT_FAIL(ctx, RT_ERR_CUDA, "%s: kernel launch failed: %s", __func__, cudaGetErrorString(_e)); \
    }                                                                                      \
  } while (0)

// After a synchronisation: reads and clears the status word; a recorded code becomes RT_ERR_TIMEOUT.
static inline rt_status rt_take_status(rt_ctx* ctx, int* code) {
  const int c = ctx->host_status ? *ctx->host_status : 0;
  if (code) *code = c;
  if (c != 0) {
    *ctx->host_status = 0;
    RT_FAIL(ctx, RT_ERR_TIMEOUT, "a kernel gave up a bounded wait (code %d): its work was skipped", c);
  }
  return RT_OK;
}

// Scratch memory from the context pool, released when the guard goes out of scope
// (stream-ordered, so the block may be reused by the next call).
struct RtScratch {
  rt_ctx* ctx;
  void* ptr = nullptr;
  explicit RtScratch(rt_ctx* c) : ctx(c) {}
  rt_status alloc(size_t bytes) { return rt_malloc(ctx, bytes, &ptr); }
  ~RtScratch() {
    if (ptr) rt_free(ctx, ptr);
  }
  template <class T>
  T* as() { return static_cast<T*>(ptr); }
};

// Runs the calls between construction and end() on the context's side stream, when the context allows it and no
// other section is open; join() (or the destructor) makes the main stream wait for them.  With `want` false, or when a
// section is already open, everything simply stays on the main stream.
struct RtFork {
  rt_ctx* ctx;
  bool open = false, pending = false;
  RtFork(rt_ctx* c, bool want);
  rt_status end();
  rt_status join();
  ~RtFork() {
    end();
    join();
  }
};

static inline int rt_grid_for(rt_ctx* ctx, int64_t work_items, int per_block, int max_waves = 8) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  int64_t cap = (int64_t)ctx->sm_count * max_waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

static __host__ __device__ inline bool rt_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
