// Context, caching allocator, copies, CUDA-graph capture, timers and the NCCL
// gradient all-reduce of librt_b200.so.
#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

// NCCL's header is only needed for the communicator configuration of the non-blocking mode (NCCL_CONFIG_INITIALIZER); the
// library itself is resolved with dlopen at run time.
#if defined(__has_include)
#if __has_include(<nccl.h>)
#include <nccl.h>
#define RT_HAVE_NCCL_HEADER 1
#endif
#endif

#include "rt_internal.cuh"

extern "C" {

int rt_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

rt_status rt_ctx_create(int device, rt_ctx** out) {
  if (!out) return RT_ERR_INVALID_OPERATION;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return RT_ERR_CUDA;  // no CUDA device: this library has no CPU fallback
  }
  if (device < 0 || device >= n) return RT_ERR_INVALID_INDEX;
  rt_ctx* ctx = new rt_ctx();
  ctx->device = device;
  if (cudaSetDevice(device) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete ctx;
    return RT_ERR_CUDA;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
  // The status word lives in pinned host memory mapped into the device's address space: a kernel whose bounded wait
  // expires stores its code there, and every call that synchronises (rt_sync, rt_memcpy_d2h, rt_event_synchronize,
  // rt_timer_stop, rt_device_status) reads it afterwards without another copy.
  void* status_host = nullptr;
  if (cudaEventCreate(&ctx->ev_start) != cudaSuccess || cudaEventCreate(&ctx->ev_stop) != cudaSuccess ||
      cudaHostAlloc(&status_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
    cudaGetLastError();
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RT_ERR_CUDA;
  }
  ctx->host_status = static_cast<volatile int*>(status_host);
  *ctx->host_status = 0;
  void* status_dev = nullptr;
  if (cudaHostGetDevicePointer(&status_dev, status_host, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(status_host);
    cudaEventDestroy(ctx->ev_start);
    cudaEventDestroy(ctx->ev_stop);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RT_ERR_CUDA;
  }
  ctx->device_status = static_cast<int*>(status_dev);
  if (cudaMalloc(&ctx->reduce_counters, 2 * (kReduceCounterSlots + kAuxCounterSlots) * sizeof(unsigned)) != cudaSuccess ||
      cudaMemset(ctx->reduce_counters, 0, 2 * (kReduceCounterSlots + kAuxCounterSlots) * sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    if (ctx->reduce_counters) cudaFree(ctx->reduce_counters);
    ctx->reduce_counters = nullptr;  // the reductions then keep to their two-launch form
  }
  const char* no_tc = getenv("RT_B200_DISABLE_TENSOR_CORES");
  if (no_tc && no_tc[0] == '1') ctx->use_tensor_cores = false;
  const char* dw_tma = getenv("RT_B200_CONV_DW_TMA");
  if (dw_tma && dw_tma[0] == '0') ctx->use_tma_weight_grad = false;
  const char* serial = getenv("RT_B200_SERIAL_BACKWARD");
  if (serial && serial[0] == '1') ctx->concurrent_backward = false;
  *out = ctx;
  return RT_OK;
}

rt_status rt_ctx_destroy(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  cudaSetDevice(ctx->device);
  if (ctx->on_side) ctx->stream = ctx->main_stream;
  cudaStreamSynchronize(ctx->stream);
  if (ctx->side_stream) {
    cudaStreamSynchronize(ctx->side_stream);
    cudaStreamDestroy(ctx->side_stream);
    cudaEventDestroy(ctx->fork_ev);
    cudaEventDestroy(ctx->join_ev);
  }
  rt_dp_finalize(ctx);
  for (auto& kv : ctx->free_blocks) cudaFree(kv.second);
  for (auto& kv : ctx->capture_free) cudaFree(kv.second);
  for (auto& kv : ctx->side_deferred) cudaFree(kv.second);
  for (auto& kv : ctx->live_blocks) cudaFree(kv.first);
  if (ctx->host_status) cudaFreeHost(const_cast<int*>(ctx->host_status));
  if (ctx->reduce_counters) cudaFree(ctx->reduce_counters);
  if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
  if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return RT_OK;
}

const char* rt_last_error(rt_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

static size_t round_size(size_t bytes) {
  if (bytes == 0) bytes = 1;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
  const size_t two_mb = size_t(2) << 20;
  return (bytes + two_mb - 1) / two_mb * two_mb;
}

rt_status rt_malloc(rt_ctx* ctx, size_t bytes, void** out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, out);
  if (ctx->on_side && !ctx->side_internal) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_malloc inside a side-stream section");
  size_t sz = round_size(bytes);
  if (ctx->capturing) {
    auto cit = ctx->capture_free.lower_bound(sz);
    if (cit != ctx->capture_free.end() && cit->first <= sz + sz / 4) {
      *out = cit->second;
      ctx->live_blocks[cit->second] = cit->first;
      ctx->bytes_in_use += (int64_t)cit->first;
      ctx->capture_free.erase(cit);
      return RT_OK;
    }
  }
  auto it = ctx->free_blocks.lower_bound(sz);
  if (it != ctx->free_blocks.end() && it->first <= sz + sz / 4) {
    *out = it->second;
    ctx->live_blocks[it->second] = it->first;
    ctx->bytes_in_use += (int64_t)it->first;
    ctx->free_blocks.erase(it);
    return RT_OK;
  }
  void* p = nullptr;
  cudaSetDevice(ctx->device);
  cudaError_t e = cudaMalloc(&p, sz);
  if (e == cudaErrorMemoryAllocation) {
    // Give cached blocks back to the driver and retry once.
    cudaGetLastError();
    if (!ctx->capturing) {
      cudaStreamSynchronize(ctx->stream);
      for (auto& kv : ctx->free_blocks) {
        cudaFree(kv.second);
        ctx->bytes_reserved -= (int64_t)kv.first;
      }
      ctx->free_blocks.clear();
      e = cudaMalloc(&p, sz);
    }
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    RT_FAIL(ctx, e == cudaErrorMemoryAllocation ? RT_ERR_OOM : RT_ERR_CUDA, "cudaMalloc(%zu) failed: %s", sz,
            cudaGetErrorString(e));
  }
  ctx->n_device_allocs++;
  ctx->bytes_reserved += (int64_t)sz;
  ctx->bytes_in_use += (int64_t)sz;
  ctx->live_blocks[p] = sz;
  *out = p;
  return RT_OK;
}

rt_status rt_free(rt_ctx* ctx, void* ptr) {
  RT_CHECK_CTX(ctx);
  if (!ptr) return RT_OK;
  auto it = ctx->live_blocks.find(ptr);
  if (it == ctx->live_blocks.end()) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_free: pointer %p is not a live block", ptr);
  ctx->bytes_in_use -= (int64_t)it->second;
  if (ctx->on_side && ctx->side_internal) ctx->side_deferred.emplace_back(it->second, ptr);
  else if (ctx->capturing) ctx->capture_free.emplace(it->second, ptr);
  else ctx->free_blocks.emplace(it->second, ptr);
  ctx->live_blocks.erase(it);
  return RT_OK;
}

rt_status rt_mem_stats(rt_ctx* ctx, int64_t* reserved, int64_t* in_use, int64_t* n_allocs) {
  RT_CHECK_CTX(ctx);
  if (reserved) *reserved = ctx->bytes_reserved;
  if (in_use) *in_use = ctx->bytes_in_use;
  if (n_allocs) *n_allocs = ctx->n_device_allocs;
  return RT_OK;
}

rt_status rt_kernel_launch_count(rt_ctx* ctx, int64_t* launches) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, launches);
  *launches = ctx->launches;
  return RT_OK;
}

rt_status rt_memcpy_h2d(rt_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RT_CHECK_CTX(ctx);
  if (bytes == 0) return RT_OK;
  RT_CHECK_PTR(ctx, dst);
  RT_CHECK_PTR(ctx, src);
  if (ctx->capturing)  // the synchronisation below would end the capture with an error of its own
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION,
            "rt_memcpy_h2d synchronises the stream and cannot be recorded in a graph: stage host data before rt_graph_begin");
  RT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  // The source may be pageable and freed by the caller right after the call.
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return RT_OK;
}

rt_status rt_memcpy_d2h(rt_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RT_CHECK_CTX(ctx);
  if (bytes == 0) return RT_OK;
  RT_CHECK_PTR(ctx, dst);
  RT_CHECK_PTR(ctx, src);
  if (ctx->capturing)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION,
            "rt_memcpy_d2h synchronises the stream and cannot be recorded in a graph (an op that reads a device value on the host, "
            "such as sqrt's negative-input check, is not capturable)");
  RT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return rt_take_status(ctx, nullptr);
}

rt_status rt_memcpy_h2d_async(rt_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RT_CHECK_CTX(ctx);
  if (bytes == 0) return RT_OK;
  RT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return RT_OK;
}

rt_status rt_memcpy_d2h_async(rt_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RT_CHECK_CTX(ctx);
  if (bytes == 0) return RT_OK;
  RT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return RT_OK;
}

rt_status rt_memcpy_d2d(rt_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RT_CHECK_CTX(ctx);
  if (bytes == 0) return RT_OK;
  RT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return RT_OK;
}

rt_status rt_host_alloc(rt_ctx* ctx, size_t bytes, void** out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, out);
  RT_CUDA(ctx, cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
  return RT_OK;
}

rt_status rt_host_free(rt_ctx* ctx, void* ptr) {
  RT_CHECK_CTX(ctx);
  if (ptr) RT_CUDA(ctx, cudaFreeHost(ptr));
  return RT_OK;
}

rt_status rt_sync(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return rt_take_status(ctx, nullptr);
}

void* rt_stream(rt_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

// ---- double-buffered input upload ------------------------------------------------------------
struct rt_upload {
  size_t bytes = 0;
  cudaStream_t copy_stream = nullptr;
  void* pinned[2] = {nullptr, nullptr};
  void* staging[2] = {nullptr, nullptr};
  cudaEvent_t copied[2] = {nullptr, nullptr};    // H2D of this pair finished (copy stream)
  cudaEvent_t consumed[2] = {nullptr, nullptr};  // staging -> dst of this pair finished (context stream)
  bool used[2] = {false, false};
  int next = 0;
};

rt_status rt_upload_destroy(rt_ctx* ctx, rt_upload* up) {
  RT_CHECK_CTX(ctx);
  if (!up) return RT_OK;
  if (up->copy_stream) cudaStreamSynchronize(up->copy_stream);
  cudaStreamSynchronize(ctx->stream);
  for (int i = 0; i < 2; ++i) {
    if (up->pinned[i]) cudaFreeHost(up->pinned[i]);
    if (up->staging[i]) cudaFree(up->staging[i]);
    if (up->copied[i]) cudaEventDestroy(up->copied[i]);
    if (up->consumed[i]) cudaEventDestroy(up->consumed[i]);
  }
  if (up->copy_stream) cudaStreamDestroy(up->copy_stream);
  delete up;
  return RT_OK;
}

rt_status rt_upload_create(rt_ctx* ctx, size_t bytes, rt_upload** out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, out);
  *out = nullptr;
  RT_CUDA(ctx, cudaSetDevice(ctx->device));  // the calling thread's current device may be another one
  rt_upload* up = new rt_upload();
  up->bytes = bytes ? bytes : 1;
  cudaError_t e = cudaStreamCreateWithFlags(&up->copy_stream, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
    e = cudaHostAlloc(&up->pinned[i], up->bytes, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaMalloc(&up->staging[i], up->bytes);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&up->copied[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&up->consumed[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    rt_upload_destroy(ctx, up);
    RT_FAIL(ctx, e == cudaErrorMemoryAllocation ? RT_ERR_OOM : RT_ERR_CUDA, "rt_upload_create: %s", cudaGetErrorString(e));
  }
  *out = up;
  return RT_OK;
}

rt_status rt_upload_host_buffer(rt_ctx* ctx, rt_upload* up, void** pinned) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, up);
  RT_CHECK_PTR(ctx, pinned);
  const int k = up->next;
  if (up->used[k]) RT_CUDA(ctx, cudaEventSynchronize(up->copied[k]));  // the copy that last read this buffer
  *pinned = up->pinned[k];
  return RT_OK;
}

rt_status rt_upload_submit(rt_ctx* ctx, rt_upload* up, void* dst) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, up);
  RT_CHECK_PTR(ctx, dst);
  if (ctx->capturing) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_upload_submit during graph capture");
  const int k = up->next;
  // the staging buffer may still be read by the staging -> dst copy of two submits ago
  if (up->used[k]) RT_CUDA(ctx, cudaStreamWaitEvent(up->copy_stream, up->consumed[k], 0));
  RT_CUDA(ctx, cudaMemcpyAsync(up->staging[k], up->pinned[k], up->bytes, cudaMemcpyHostToDevice, up->copy_stream));
  RT_CUDA(ctx, cudaEventRecord(up->copied[k], up->copy_stream));
  RT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, up->copied[k], 0));
  RT_CUDA(ctx, cudaMemcpyAsync(dst, up->staging[k], up->bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  RT_CUDA(ctx, cudaEventRecord(up->consumed[k], ctx->stream));
  up->used[k] = true;
  up->next = k ^ 1;
  return RT_OK;
}

// ---- several uploads in one go, and a result written straight to pinned host memory ---------------
// A training step that takes its inputs from the host needs, per step, one staging -> tensor copy per input and the
// read-back of the loss.  As stream memcpys these are three copy-engine round trips between two graph launches; as
// two small kernels they run back to back with the step's own kernels.
constexpr int kMaxUploadsPerSubmit = 8;
struct MultiCopyParams {
  const char* src[kMaxUploadsPerSubmit];
  char* dst[kMaxUploadsPerSubmit];
  unsigned long long bytes[kMaxUploadsPerSubmit];
};
// blockIdx.y = which copy; 16-byte units when both ends are 16-byte aligned, single bytes for the rest
__global__ void multi_copy_kernel(const MultiCopyParams p) {
  const int seg = blockIdx.y;
  const char* __restrict__ src = p.src[seg];
  char* __restrict__ dst = p.dst[seg];
  const size_t bytes = p.bytes[seg];
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  size_t done = 0;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const size_t n16 = bytes >> 4;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (size_t i = tid; i < n16; i += nthreads) d4[i] = __ldcs(s4 + i);
    done = n16 << 4;
  }
  for (size_t i = done + tid; i < bytes; i += nthreads) dst[i] = src[i];
}

rt_status rt_upload_submit_all(rt_ctx* ctx, rt_upload* const* ups, void* const* dsts, int n) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, ups);
  RT_CHECK_PTR(ctx, dsts);
  if (n < 1 || n > kMaxUploadsPerSubmit)
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_upload_submit_all: 1 to %d uploads per call, got %d", kMaxUploadsPerSubmit, n);
  if (ctx->capturing) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_upload_submit_all during graph capture");
  for (int i = 0; i < n; ++i) {
    RT_CHECK_PTR(ctx, ups[i]);
    RT_CHECK_PTR(ctx, dsts[i]);
    for (int j = 0; j < i; ++j)
      if (ups[j] == ups[i]) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_upload_submit_all: upload %d is listed twice", i);
  }
  MultiCopyParams p{};
  size_t most = 0;
  for (int i = 0; i < n; ++i) {
    rt_upload* up = ups[i];
    const int k = up->next;
    // the staging buffer may still be read by the staging -> dst copy of two submits ago
    if (up->used[k]) RT_CUDA(ctx, cudaStreamWaitEvent(up->copy_stream, up->consumed[k], 0));
    RT_CUDA(ctx, cudaMemcpyAsync(up->staging[k], up->pinned[k], up->bytes, cudaMemcpyHostToDevice, up->copy_stream));
    RT_CUDA(ctx, cudaEventRecord(up->copied[k], up->copy_stream));
    RT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, up->copied[k], 0));
    p.src[i] = static_cast<const char*>(up->staging[k]);
    p.dst[i] = static_cast<char*>(dsts[i]);
    p.bytes[i] = up->bytes;
    most = up->bytes > most ? up->bytes : most;
  }
  const size_t units = (most + 15) / 16;
  const unsigned blocks = (unsigned)std::min<size_t>((units + 255) / 256, (size_t)ctx->sm_count * 4);
  multi_copy_kernel<<<dim3(blocks ? blocks : 1, (unsigned)n), 256, 0, ctx->stream>>>(p);
  RT_LAUNCHED(ctx);
  for (int i = 0; i < n; ++i) {
    rt_upload* up = ups[i];
    const int k = up->next;
    RT_CUDA(ctx, cudaEventRecord(up->consumed[k], ctx->stream));
    up->used[k] = true;
    up->next = k ^ 1;
  }
  return RT_OK;
}

__global__ void publish_kernel(const float* __restrict__ src, float* __restrict__ host_dst, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) host_dst[i] = src[i];
  __threadfence_system();
}

rt_status rt_publish_to_host(rt_ctx* ctx, float* pinned_dst, const float* src, int64_t n) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, pinned_dst);
  RT_CHECK_PTR(ctx, src);
  if (n < 1 || n > 4096) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_publish_to_host: 1 to 4096 values, got %lld", (long long)n);
  // The kernel stores through the host pointer, so it must be pinned memory the device can reach (rt_host_alloc).
  cudaPointerAttributes attr{};
  cudaError_t e = cudaPointerGetAttributes(&attr, pinned_dst);
  if (e != cudaSuccess || attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) {
    if (e != cudaSuccess) cudaGetLastError();
    RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_publish_to_host: the destination is not pinned host memory (use rt_host_alloc)");
  }
  publish_kernel<<<1, n < 256 ? 32 : 256, 0, ctx->stream>>>(src, static_cast<float*>(attr.devicePointer), (int)n);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// ---- side stream --------------------------------------------------------------------------------
rt_status rt_side_stream_begin(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  if (ctx->on_side) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_side_stream_begin: a side section is already open");
  if (ctx->side_pending) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_side_stream_begin: join the previous side section first");
  if (!ctx->side_stream) {
    RT_CUDA(ctx, cudaSetDevice(ctx->device));
    RT_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    RT_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming));
    RT_CUDA(ctx, cudaEventCreateWithFlags(&ctx->join_ev, cudaEventDisableTiming));
  }
  RT_CUDA(ctx, cudaEventRecord(ctx->fork_ev, ctx->stream));
  RT_CUDA(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->fork_ev, 0));
  ctx->main_stream = ctx->stream;
  ctx->stream = ctx->side_stream;
  ctx->on_side = true;
  return RT_OK;
}
rt_status rt_side_stream_end(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  if (!ctx->on_side) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_side_stream_end: no side section is open");
  cudaError_t e = cudaEventRecord(ctx->join_ev, ctx->side_stream);
  ctx->stream = ctx->main_stream;
  ctx->on_side = false;
  ctx->side_pending = true;
  RT_CUDA(ctx, e);
  return RT_OK;
}
rt_status rt_side_stream_join(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  if (ctx->on_side) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_side_stream_join: end the side section first");
  if (!ctx->side_pending) return RT_OK;
  ctx->side_pending = false;
  RT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->join_ev, 0));
  return RT_OK;
}

RtFork::RtFork(rt_ctx* c, bool want) : ctx(c) {
  if (!want || !c->concurrent_backward || c->on_side || c->side_pending) return;
  if (rt_side_stream_begin(c) != RT_OK) return;
  c->side_internal = true;
  open = true;
}
rt_status RtFork::end() {
  if (!open) return RT_OK;
  open = false;
  pending = true;
  ctx->side_internal = false;
  return rt_side_stream_end(ctx);
}
rt_status RtFork::join() {
  if (!pending) return RT_OK;
  pending = false;
  rt_status st = rt_side_stream_join(ctx);
  // ordered after the join on the main stream: the parked blocks may be handed out again
  for (auto& kv : ctx->side_deferred) {
    if (ctx->capturing) ctx->capture_free.emplace(kv.first, kv.second);
    else ctx->free_blocks.emplace(kv.first, kv.second);
  }
  ctx->side_deferred.clear();
  return st;
}

// ---- events on the context's stream -----------------------------------------------------------
struct rt_event {
  cudaEvent_t ev = nullptr;
};
rt_status rt_event_create(rt_ctx* ctx, rt_event** out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, out);
  RT_CUDA(ctx, cudaSetDevice(ctx->device));
  rt_event* e = new rt_event();
  cudaError_t err = cudaEventCreateWithFlags(&e->ev, cudaEventDisableTiming);
  if (err != cudaSuccess) {
    delete e;
    RT_FAIL(ctx, RT_ERR_CUDA, "rt_event_create: %s", cudaGetErrorString(err));
  }
  *out = e;
  return RT_OK;
}
rt_status rt_event_destroy(rt_ctx* ctx, rt_event* ev) {
  RT_CHECK_CTX(ctx);
  if (ev) {
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
  }
  return RT_OK;
}
rt_status rt_event_record(rt_ctx* ctx, rt_event* ev) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, ev);
  RT_CUDA(ctx, cudaEventRecord(ev->ev, ctx->stream));
  return RT_OK;
}
rt_status rt_event_synchronize(rt_ctx* ctx, rt_event* ev) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, ev);
  RT_CUDA(ctx, cudaEventSynchronize(ev->ev));
  return rt_take_status(ctx, nullptr);
}

rt_status rt_device_status(rt_ctx* ctx, int* code) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, code);
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return rt_take_status(ctx, code);
}

rt_status rt_set_tensor_cores(rt_ctx* ctx, int enable) {
  RT_CHECK_CTX(ctx);
  ctx->use_tensor_cores = enable != 0;
  return RT_OK;
}

rt_status rt_set_concurrent_backward(rt_ctx* ctx, int enable) {
  RT_CHECK_CTX(ctx);
  ctx->concurrent_backward = enable != 0;
  return RT_OK;
}

// ---- CUDA graphs -----------------------------------------------------------------
rt_status rt_graph_begin(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  if (ctx->capturing) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_graph_begin: already capturing");
  // Relaxed mode: the pool may still call cudaMalloc for a size it has not seen.
  RT_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = true;
  return RT_OK;
}

rt_status rt_graph_end(rt_ctx* ctx, rt_graph** out) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, out);
  if (!ctx->capturing) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "rt_graph_end: not capturing");
  ctx->capturing = false;
  rt_graph* g = new rt_graph();
  for (auto& kv : ctx->capture_free) g->retired.emplace_back(kv.first, kv.second);
  ctx->capture_free.clear();
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (g->graph) cudaGraphDestroy(g->graph);
    for (auto& kv : g->retired) ctx->free_blocks.emplace(kv.first, kv.second);
    delete g;
    RT_FAIL(ctx, RT_ERR_CUDA, "graph capture/instantiate failed: %s", cudaGetErrorString(e));
  }
  *out = g;
  return RT_OK;
}

rt_status rt_graph_launch(rt_ctx* ctx, rt_graph* g) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, g);
  RT_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  return RT_OK;
}

rt_status rt_graph_num_nodes(rt_ctx* ctx, rt_graph* g, int64_t* n) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, g);
  size_t cnt = 0;
  RT_CUDA(ctx, cudaGraphGetNodes(g->graph, nullptr, &cnt));
  *n = (int64_t)cnt;
  return RT_OK;
}

rt_status rt_graph_destroy(rt_ctx* ctx, rt_graph* g) {
  RT_CHECK_CTX(ctx);
  if (!g) return RT_OK;
  cudaStreamSynchronize(ctx->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  for (auto& kv : g->retired) ctx->free_blocks.emplace(kv.first, kv.second);
  delete g;
  return RT_OK;
}

// ---- timers ----------------------------------------------------------------------
rt_status rt_timer_start(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  RT_CUDA(ctx, cudaEventRecord(ctx->ev_start, ctx->stream));
  return RT_OK;
}

rt_status rt_timer_stop(rt_ctx* ctx, float* ms) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, ms);
  RT_CUDA(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream));
  RT_CUDA(ctx, cudaEventSynchronize(ctx->ev_stop));
  RT_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_start, ctx->ev_stop));
  return rt_take_status(ctx, nullptr);
}

__global__ void stamp_kernel(unsigned long long* dst) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  *dst = t;
}
rt_status rt_stamp(rt_ctx* ctx, uint64_t* dst) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, dst);
  stamp_kernel<<<1, 1, 0, ctx->stream>>>(reinterpret_cast<unsigned long long*>(dst));
  RT_LAUNCHED(ctx);
  return RT_OK;
}

// ---- NCCL, resolved at run time so that the library loads on machines without it ---
// RT_B200_NCCL_LIBRARY names the shared object to load instead of libnccl.so.2 (the failure-handling tests load a
// scripted stand-in through it).
namespace {
struct NcclId {
  char internal[128];
};
constexpr int kNcclSuccess = 0, kNcclInProgress = 7;
struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
  int (*CommInitRankConfig)(void**, int, NcclId, int, void*) = nullptr;
  int (*CommGetAsyncError)(void*, int*) = nullptr;
  int (*CommAbort)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
  const char* text(int rc) const { return GetErrorString ? GetErrorString(rc) : "?"; }
};
NcclApi& nccl() {
  static NcclApi api;
  if (!api.handle) {
    const char* custom = getenv("RT_B200_NCCL_LIBRARY");
    if (custom && custom[0]) {
      api.handle = dlopen(custom, RTLD_NOW | RTLD_GLOBAL);
    } else {
      api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    }
    if (api.handle) {
      api.GetUniqueId = (int (*)(NcclId*))dlsym(api.handle, "ncclGetUniqueId");
      api.CommInitRank = (int (*)(void**, int, NcclId, int))dlsym(api.handle, "ncclCommInitRank");
      api.CommInitRankConfig = (int (*)(void**, int, NcclId, int, void*))dlsym(api.handle, "ncclCommInitRankConfig");
      api.CommGetAsyncError = (int (*)(void*, int*))dlsym(api.handle, "ncclCommGetAsyncError");
      api.CommAbort = (int (*)(void*))dlsym(api.handle, "ncclCommAbort");
      api.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(api.handle, "ncclAllReduce");
      api.CommDestroy = (int (*)(void*))dlsym(api.handle, "ncclCommDestroy");
      api.GetErrorString = (const char* (*)(int))dlsym(api.handle, "ncclGetErrorString");
      api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy;
    }
  }
  return api;
}

int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Gives the communicator up after a failure: ncclCommAbort also ends collective kernels that are stuck on a missing peer.
void abandon_comm(rt_ctx* ctx, void* comm) {
  NcclApi& n = nccl();
  if (comm) {
    if (n.CommAbort) n.CommAbort(comm);
    else n.CommDestroy(comm);
  }
  if (ctx->nccl_comm == comm) ctx->nccl_comm = nullptr;
}

// Polls the communicator until its pending call has finished.  RT_OK, RT_ERR_NCCL (the communicator reported an error) or
// RT_ERR_TIMEOUT (the deadline passed first); after either error the communicator has been aborted.
rt_status settle_comm(rt_ctx* ctx, void* comm, const char* what) {
  NcclApi& n = nccl();
  const int64_t deadline = now_ms() + ctx->dp_timeout_ms;
  for (int spins = 0;; ++spins) {
    int state = kNcclSuccess;
    const int rc = n.CommGetAsyncError(comm, &state);
    if (rc != kNcclSuccess) {
      abandon_comm(ctx, comm);
      RT_FAIL(ctx, RT_ERR_NCCL, "%s: ncclCommGetAsyncError failed: %s", what, n.text(rc));
    }
    if (state == kNcclSuccess) return RT_OK;
    if (state != kNcclInProgress) {
      abandon_comm(ctx, comm);
      RT_FAIL(ctx, RT_ERR_NCCL, "%s: the communicator reported: %s", what, n.text(state));
    }
    if (now_ms() > deadline) {
      abandon_comm(ctx, comm);
      RT_FAIL(ctx, RT_ERR_TIMEOUT, "%s: not finished after %lld ms (a rank that never joined?); communicator aborted", what,
              (long long)ctx->dp_timeout_ms);
    }
    if (spins > 1000) std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}
}  // namespace

rt_status rt_dp_unique_id(uint8_t id[RT_DP_ID_BYTES]) {
  if (!id) return RT_ERR_INVALID_OPERATION;
  NcclApi& n = nccl();
  if (!n.ok) return RT_ERR_NCCL;
  NcclId nid;
  if (n.GetUniqueId(&nid) != 0) return RT_ERR_NCCL;
  static_assert(sizeof(NcclId) == RT_DP_ID_BYTES, "id size");
  memcpy(id, &nid, sizeof(nid));
  return RT_OK;
}

rt_status rt_dp_init_deadline(rt_ctx* ctx, int rank, int world, const uint8_t id[RT_DP_ID_BYTES], int64_t timeout_ms) {
  RT_CHECK_CTX(ctx);
  if (world < 1 || rank < 0 || rank >= world) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "rt_dp_init: rank %d of %d", rank, world);
  ctx->dp_rank = rank;
  ctx->dp_world = world;
  if (world == 1) return RT_OK;
  if (ctx->nccl_comm) return RT_OK;  // already joined (a second trainer on the same context reuses the communicator)
  RT_CHECK_PTR(ctx, id);
  NcclApi& n = nccl();
  if (!n.ok) RT_FAIL(ctx, RT_ERR_NCCL, "the NCCL library could not be loaded");
  NcclId nid;
  memcpy(&nid, id, sizeof(nid));
  RT_CUDA(ctx, cudaSetDevice(ctx->device));
  bool nonblocking = timeout_ms > 0 && n.CommInitRankConfig && n.CommGetAsyncError && n.CommAbort;
#ifndef RT_HAVE_NCCL_HEADER
  nonblocking = false;  // the configuration structure comes from NCCL's own header
#endif
  if (!nonblocking) {
    const int rc = n.CommInitRank(&ctx->nccl_comm, world, nid, rank);
    if (rc != kNcclSuccess) {
      ctx->nccl_comm = nullptr;
      RT_FAIL(ctx, RT_ERR_NCCL, "ncclCommInitRank failed: %s", n.text(rc));
    }
    ctx->nccl_nonblocking = false;
    return RT_OK;
  }
#ifdef RT_HAVE_NCCL_HEADER
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;
  void* comm = nullptr;
  const int rc = n.CommInitRankConfig(&comm, world, nid, rank, &config);
  if (rc != kNcclSuccess && rc != kNcclInProgress) {
    if (comm) abandon_comm(ctx, comm);
    RT_FAIL(ctx, RT_ERR_NCCL, "ncclCommInitRankConfig failed: %s", n.text(rc));
  }
  if (!comm) RT_FAIL(ctx, RT_ERR_NCCL, "ncclCommInitRankConfig returned no communicator");
  ctx->dp_timeout_ms = timeout_ms;
  const rt_status st = settle_comm(ctx, comm, "rt_dp_init");
  if (st != RT_OK) return st;
  ctx->nccl_comm = comm;
  ctx->nccl_nonblocking = true;
#endif
  return RT_OK;
}

rt_status rt_dp_init(rt_ctx* ctx, int rank, int world, const uint8_t id[RT_DP_ID_BYTES]) {
  // Blocking communicator by default: on a non-blocking one every ncclAllReduce answers "in progress" and has to be polled,
  // which measured 0.13 ms of host time per step on eight B200s (end-to-end step 0.46 ms against 0.33 ms).  Callers that
  // want the join bounded use rt_dp_init_deadline or set RT_B200_NCCL_NONBLOCKING=1 (deadline RT_B200_DP_TIMEOUT_MS,
  // default 120000); the asynchronous-error watchdog (rt_dp_async_error, rt_dp_wait_event) works on either kind.
  int64_t timeout_ms = 0;
  const char* nb = getenv("RT_B200_NCCL_NONBLOCKING");
  if (nb && nb[0] == '1') {
    timeout_ms = 120000;
    const char* env = getenv("RT_B200_DP_TIMEOUT_MS");
    if (env && env[0]) timeout_ms = atoll(env);
  }
  return rt_dp_init_deadline(ctx, rank, world, id, timeout_ms);
}

rt_status rt_dp_allreduce_sum(rt_ctx* ctx, float* buf, int64_t count) {
  RT_CHECK_CTX(ctx);
  if (ctx->dp_world == 1 || count == 0) return RT_OK;
  RT_CHECK_PTR(ctx, buf);
  if (!ctx->nccl_comm) RT_FAIL(ctx, RT_ERR_NCCL, "rt_dp_allreduce_sum: no communicator (rt_dp_init was not called, or it was aborted)");
  NcclApi& n = nccl();
  const int nccl_float32 = 7, nccl_sum = 0;
  const int rc = n.AllReduce(buf, buf, (size_t)count, nccl_float32, nccl_sum, ctx->nccl_comm, ctx->stream);
  if (rc == kNcclInProgress && ctx->nccl_nonblocking) return settle_comm(ctx, ctx->nccl_comm, "rt_dp_allreduce_sum");
  if (rc != kNcclSuccess) RT_FAIL(ctx, RT_ERR_NCCL, "ncclAllReduce failed: %s", n.text(rc));
  return RT_OK;
}

rt_status rt_dp_async_error(rt_ctx* ctx, int* nccl_code) {
  RT_CHECK_CTX(ctx);
  if (nccl_code) *nccl_code = 0;
  NcclApi& n = nccl();
  if (!ctx->nccl_comm || !n.CommGetAsyncError) return RT_OK;
  int state = kNcclSuccess;
  const int rc = n.CommGetAsyncError(ctx->nccl_comm, &state);
  if (rc != kNcclSuccess) state = rc;
  if (nccl_code) *nccl_code = state;
  if (state == kNcclSuccess || state == kNcclInProgress) return RT_OK;
  abandon_comm(ctx, ctx->nccl_comm);
  RT_FAIL(ctx, RT_ERR_NCCL, "the communicator reported an asynchronous error: %s; communicator aborted", n.text(state));
}

rt_status rt_dp_wait_event(rt_ctx* ctx, rt_event* ev) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, ev);
  if (!ctx->nccl_comm) return rt_event_synchronize(ctx, ev);
  const int64_t deadline = now_ms() + ctx->dp_timeout_ms;
  for (int spins = 0;; ++spins) {
    const cudaError_t q = cudaEventQuery(ev->ev);
    if (q == cudaSuccess) return rt_take_status(ctx, nullptr);
    if (q != cudaErrorNotReady) RT_FAIL(ctx, RT_ERR_CUDA, "rt_dp_wait_event: %s", cudaGetErrorString(q));
    if ((spins & 63) == 63) {
      const rt_status st = rt_dp_async_error(ctx, nullptr);
      if (st != RT_OK) return st;
      if (now_ms() > deadline) {
        abandon_comm(ctx, ctx->nccl_comm);
        RT_FAIL(ctx, RT_ERR_TIMEOUT, "rt_dp_wait_event: the step did not finish within %lld ms; communicator aborted",
                (long long)ctx->dp_timeout_ms);
      }
    }
    if (spins > 20000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

rt_status rt_ipc_export(rt_ctx* ctx, void* device_ptr, uint8_t handle[RT_IPC_HANDLE_BYTES]) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, device_ptr);
  RT_CHECK_PTR(ctx, handle);
  static_assert(sizeof(cudaIpcMemHandle_t) == RT_IPC_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  RT_CUDA(ctx, cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle, &h, sizeof(h));
  return RT_OK;
}
rt_status rt_ipc_open(rt_ctx* ctx, const uint8_t handle[RT_IPC_HANDLE_BYTES], void** peer_ptr) {
  RT_CHECK_CTX(ctx);
  RT_CHECK_PTR(ctx, handle);
  RT_CHECK_PTR(ctx, peer_ptr);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  RT_CUDA(ctx, cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return RT_OK;
}
rt_status rt_ipc_close(rt_ctx* ctx, void* peer_ptr) {
  RT_CHECK_CTX(ctx);
  if (peer_ptr) RT_CUDA(ctx, cudaIpcCloseMemHandle(peer_ptr));
  return RT_OK;
}

rt_status rt_dp_finalize(rt_ctx* ctx) {
  RT_CHECK_CTX(ctx);
  if (ctx->nccl_comm) {
    cudaStreamSynchronize(ctx->stream);  // no collective of this communicator is still queued
    nccl().CommDestroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
    ctx->nccl_nonblocking = false;
  }
  ctx->dp_world = 1;
  ctx->dp_rank = 0;
  return RT_OK;
}

}  // extern "C"
