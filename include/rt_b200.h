/*
 * rt_b200.h -- C ABI of the sm_100a backward-pass backend.
 *
 * Every entry point takes plain pointers and sizes.  All `float*` / `void*` data
 * arguments are DEVICE pointers unless the name says `host`.  All tensors are fp32,
 * row-major, contiguous (NCHW for images); a 0-dimensional tensor is one element.
 * Calls are asynchronous on the context's stream unless stated otherwise; nothing
 * here synchronises except rt_sync, rt_memcpy_d2h and rt_sum_all_host.
 *
 * Each declaration cites the method of the reference's `Backend` trait
 * (src/backend/mod.rs) -- or the helper it calls -- that a Rust
 * `impl Backend for B200Backend` would forward to it.
 *
 * Return value: RT_OK or one of the RT_ERR_* codes, which mirror the variants of the
 * reference's `Error` enum (src/error.rs:8-98).  rt_last_error(ctx) gives the text.
 */
#ifndef RT_B200_H
#define RT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rt_ctx rt_ctx;     /* one device + one stream + a caching allocator (+ an NCCL communicator) */
typedef struct rt_graph rt_graph; /* an instantiated CUDA graph of a captured call sequence */
typedef int32_t rt_status;

enum {
  RT_OK = 0,
  RT_ERR_SHAPE_MISMATCH = 1,      /* Error::ShapeMismatch */
  RT_ERR_INCOMPATIBLE_SHAPES = 2, /* Error::IncompatibleShapes */
  RT_ERR_INVALID_INDEX = 3,       /* Error::InvalidIndex */
  RT_ERR_INVALID_OPERATION = 4,   /* Error::InvalidOperation */
  RT_ERR_INTERNAL = 5,            /* Error::InternalLogicError */
  RT_ERR_DIMENSION_MISMATCH = 6,  /* Error::DimensionMismatch */
  RT_ERR_CUDA = 7,                /* Error::CudaError */
  RT_ERR_OOM = 8,                 /* Error::OutOfMemory */
  RT_ERR_UNIMPLEMENTED = 9,       /* Error::Unimplemented */
  RT_ERR_EMPTY_TENSOR = 10,       /* Error::EmptyTensor */
  RT_ERR_TIMEOUT = 14,            /* a bounded device-side wait gave up */
  RT_ERR_NCCL = 15,
  RT_ERR_INITIALIZATION = 16      /* Error::InitializationError (invalid parameters of a random factory) */
};

#define RT_MAX_DIMS 8

/* ---- lifecycle, memory, stream ------------------------------------------------------------
 * Replaces the reference's global CUDA context / stream / per-op cuMemAlloc
 * (src/backend/cuda/context.rs:21-34,250-306; src/backend/cuda/storage.rs:165-179). */
rt_status rt_ctx_create(int device, rt_ctx** out);
rt_status rt_ctx_destroy(rt_ctx* ctx);
const char* rt_last_error(rt_ctx* ctx);
int rt_device_count(void);
rt_status rt_malloc(rt_ctx* ctx, size_t bytes, void** out);   /* pooled; Backend::zeros/from_vec storage */
rt_status rt_free(rt_ctx* ctx, void* ptr);                    /* returns the block to the pool (stream-ordered) */
rt_status rt_memcpy_h2d(rt_ctx* ctx, void* dst, const void* host_src, size_t bytes); /* Backend::from_vec, update_from_host (mod.rs:48,252) */
rt_status rt_memcpy_d2h(rt_ctx* ctx, void* host_dst, const void* src, size_t bytes); /* Backend::copy_to_host (mod.rs:248); synchronises */
rt_status rt_memcpy_h2d_async(rt_ctx* ctx, void* dst, const void* pinned_src, size_t bytes);
rt_status rt_memcpy_d2h_async(rt_ctx* ctx, void* pinned_dst, const void* src, size_t bytes);
rt_status rt_memcpy_d2d(rt_ctx* ctx, void* dst, const void* src, size_t bytes);
rt_status rt_fill(rt_ctx* ctx, float* dst, float value, int64_t n);                  /* Backend::zeros / ones (mod.rs:44,46) */
/* Random factories: random_uniform mod.rs:63 (U[low, high)), random_normal mod.rs:66 (N(mean, std_dev^2)), bernoulli mod.rs:69
 * (1.0 with probability p), kaiming_uniform mod.rs:57 = uniform with bound sqrt(6 / fan_in) (src/init.rs:26-32).  Element i
 * is a pure function of (seed, offset + i / 4) (Philox-4x32-10): a call consumes (n + 3) / 4 counter values; the caller
 * advances `offset` by that much to continue the stream.  Invalid parameters -> RT_ERR_INITIALIZATION, as rand's
 * Uniform::new / Normal::new / Bernoulli::new fail in the reference. */
rt_status rt_random_uniform(rt_ctx* ctx, float* out, int64_t n, float low, float high, uint64_t seed, uint64_t offset);
rt_status rt_random_normal(rt_ctx* ctx, float* out, int64_t n, float mean, float std_dev, uint64_t seed, uint64_t offset);
rt_status rt_bernoulli(rt_ctx* ctx, float* out, int64_t n, float p, uint64_t seed, uint64_t offset);
rt_status rt_host_alloc(rt_ctx* ctx, size_t bytes, void** out);                      /* pinned host memory */
rt_status rt_host_free(rt_ctx* ctx, void* ptr);
rt_status rt_sync(rt_ctx* ctx);
/* ---- overlapping the next step's input upload with the running step (new; the reference uploads synchronously
 * in Backend::from_vec).  An rt_upload owns two pinned host buffers and two device staging buffers of `bytes` each
 * and a copy stream.  rt_upload_host_buffer returns the pinned buffer to fill for the next submit (it first waits
 * until the copy that last read this buffer has finished).  rt_upload_submit copies it to its staging buffer on the
 * copy stream, makes the context's stream wait for that copy, then copies staging -> dst on the context's stream and
 * switches to the other buffer pair.  Work already queued on the context's stream that reads `dst` is not disturbed,
 * so the host can submit step i+1 while step i is still running. */
typedef struct rt_upload rt_upload;
rt_status rt_upload_create(rt_ctx* ctx, size_t bytes, rt_upload** out);
rt_status rt_upload_destroy(rt_ctx* ctx, rt_upload* up);
rt_status rt_upload_host_buffer(rt_ctx* ctx, rt_upload* up, void** pinned);
rt_status rt_upload_submit(rt_ctx* ctx, rt_upload* up, void* dst);
/* The same for up to 8 uploads at once (all inputs of a step): their host -> staging copies run on their copy streams as above,
 * and ONE kernel on the context's stream copies every staging buffer to its destination, instead of one device-to-device
 * memcpy per input.  ups[i] must be distinct. */
rt_status rt_upload_submit_all(rt_ctx* ctx, rt_upload* const* ups, void* const* dsts, int n);
/* Writes n <= 4096 floats at src (device) to pinned host memory from rt_host_alloc with a one-block kernel on the context's
 * stream: the read-back of a loss (Backend::copy_to_host, mod.rs:248, without its synchronisation) costs a kernel launch
 * instead of a copy-engine round trip.  The values are visible to the host once an event recorded after this call has
 * completed.  Any other kind of destination is refused. */
rt_status rt_publish_to_host(rt_ctx* ctx, float* pinned_dst, const float* src, int64_t n);
/* A side stream for work that may overlap what follows on the context's stream (new; used to all-reduce the
 * gradients that are ready while the rest of the backward pass runs).  Between begin and end every rt_* call of this
 * context is enqueued on the side stream, which first waits for everything queued before `begin`; `join` makes the
 * context's stream wait for the side work.  Calls inside a section opened through this API must not allocate (rt_malloc fails there; the sections the library
 * opens itself inside a backward call park their frees until the join instead);
 * sections do not nest; a section opened during graph capture must be joined before the capture ends. */
rt_status rt_side_stream_begin(rt_ctx* ctx);
rt_status rt_side_stream_end(rt_ctx* ctx);
rt_status rt_side_stream_join(rt_ctx* ctx);
/* Events on the context's stream: record after queued work, wait on the host later. */
typedef struct rt_event rt_event;
rt_status rt_event_create(rt_ctx* ctx, rt_event** out);
rt_status rt_event_destroy(rt_ctx* ctx, rt_event* ev);
rt_status rt_event_record(rt_ctx* ctx, rt_event* ev);
rt_status rt_event_synchronize(rt_ctx* ctx, rt_event* ev);
void* rt_stream(rt_ctx* ctx);                                                        /* the cudaStream_t */
rt_status rt_mem_stats(rt_ctx* ctx, int64_t* bytes_reserved, int64_t* bytes_in_use, int64_t* n_device_allocs);
rt_status rt_kernel_launch_count(rt_ctx* ctx, int64_t* launches);                    /* kernels launched by this library so far */
/* Synchronises and reads the device error word: kernels that wait on barriers give up after a bounded
 * number of polls, record a code there and return; non-zero -> RT_ERR_TIMEOUT (and the word is cleared). */
rt_status rt_device_status(rt_ctx* ctx, int* code);
/* 1 (default): large contractions run on the tcgen05 3xTF32 tensor-core kernels; 0: exact FP32 kernels only. */
rt_status rt_set_tensor_cores(rt_ctx* ctx, int enable);
/* 1 (default): the independent halves of one backward call (da / db of a matmul; the bias and weight gradients of a
 * convolution beside its input gradient) are issued on two streams; 0: one after the other on the context's stream.
 * Results are bit-identical either way.  No counterpart in the reference (a scheduling switch of this backend). */
rt_status rt_set_concurrent_backward(rt_ctx* ctx, int enable);

/* Measurement aid (no counterpart in the reference): SM cycles that one tcgen05.mma.kind::tf32 of shape M x N x 8
 * occupies the tensor pipe when `iters` of them are issued back to back by one CTA (M = 64 or 128, N <= 256).
 * a_in_tmem != 0 takes the A operand from tensor memory instead of shared memory.  issue_cycles = time to issue,
 * complete_cycles = time until the last one has completed, both divided by iters.  Synchronises. */
rt_status rt_tc_issue_rate(rt_ctx* ctx, int m, int n, int a_in_tmem, int iters, double* issue_cycles, double* complete_cycles);

/* CUDA-graph capture of a fixed call sequence (one training step). */
rt_status rt_graph_begin(rt_ctx* ctx);
rt_status rt_graph_end(rt_ctx* ctx, rt_graph** out);
rt_status rt_graph_launch(rt_ctx* ctx, rt_graph* g);
rt_status rt_graph_destroy(rt_ctx* ctx, rt_graph* g);
rt_status rt_graph_num_nodes(rt_ctx* ctx, rt_graph* g, int64_t* n);

/* Device-side timing on the context's stream (CUDA events). */
rt_status rt_timer_start(rt_ctx* ctx);
rt_status rt_timer_stop(rt_ctx* ctx, float* elapsed_ms); /* synchronises */
/* A one-thread kernel that stores the GPU's nanosecond timer (%globaltimer) into *dst (device memory) when it runs: a
 * time stamp between two kernels of a stream, usable inside a captured graph, where events cannot be read back. */
rt_status rt_stamp(rt_ctx* ctx, uint64_t* dst);

/* ---- unary elementwise: y = f(x) and dx = g * f'(x), f' recomputed from the INPUT x ---------- */
enum {
  RT_RELU = 0,     /* relu mod.rs:303 / relu_backward mod.rs:344 (mask x > 0) */
  RT_ELU = 1,      /* elu mod.rs:311 / elu_backward mod.rs:356; p0 = alpha */
  RT_EXP = 2,      /* exp mod.rs:279 / exp_backward mod.rs:381 */
  RT_LN = 3,       /* ln mod.rs:281 / ln_backward mod.rs:387 */
  RT_SIN = 4,      /* sin mod.rs:474 / sin_backward mod.rs:480 */
  RT_TANH = 5,     /* tanh mod.rs:414 / tanh_backward mod.rs:420 */
  RT_SIGMOID = 6,  /* sigmoid mod.rs:305 / sigmoid_backward mod.rs:314 */
  RT_SOFTPLUS = 7, /* softplus mod.rs:426 / softplus_backward mod.rs:429 (ln(1+e^x), as the CPU backend) */
  RT_SQUARE = 8,   /* square mod.rs:444 / square_backward mod.rs:450 */
  RT_SQRT = 9,     /* sqrt mod.rs:403 / sqrt_backward mod.rs:405 */
  RT_ABS = 10,     /* abs mod.rs:395 / abs_backward mod.rs:397 */
  RT_CLIP = 11,    /* clip mod.rs:629 / clip_backward mod.rs:642; p0 = min, p1 = max (inclusive mask) */
  RT_MUL_SCALAR = 12, /* mul_scalar mod.rs:655; backward is mul_scalar on the gradient; p0 = scalar */
  RT_DIV_SCALAR = 13, /* div_scalar mod.rs:242; p0 = scalar (0 -> RT_ERR_INVALID_OPERATION) */
  RT_COS = 14,     /* cos mod.rs:486 / cos_backward mod.rs:492 */
  RT_TAN = 15,     /* tan mod.rs:498 / tan_backward mod.rs:504 */
  RT_UNARY_COUNT = 16
};
rt_status rt_unary(rt_ctx* ctx, int op, const float* x, float* y, int64_t n, float p0, float p1);
rt_status rt_unary_backward(rt_ctx* ctx, int op, const float* x, const float* g, float* dx, int64_t n, float p0, float p1);

/* ---- binary elementwise with numpy broadcasting --------------------------------------------
 * Shapes are right-aligned; out has the broadcast shape.  rt_binary_backward fuses the
 * `unbroadcast` reduction (src/ops/cpu_backward.rs:523-678) into the gradient kernels: da has
 * a's shape and db has b's shape.  Pass NULL for a gradient that is not needed. */
enum {
  RT_ADD = 0,     /* add mod.rs:236 / add_backward mod.rs:334 */
  RT_SUB = 1,     /* sub mod.rs:238 / sub_backward mod.rs:375 */
  RT_MUL = 2,     /* mul mod.rs:234 / mul_backward mod.rs:329 */
  RT_DIV = 3,     /* div mod.rs:240 / div_backward mod.rs:369 */
  RT_POWF = 4,    /* powf mod.rs:435 / powf_backward mod.rs:438 */
  RT_MAXIMUM = 5, /* maximum mod.rs:456 / maximum_backward mod.rs:459 (ties -> a) */
  RT_MINIMUM = 6, /* minimum mod.rs:465 / minimum_backward mod.rs:468 (ties -> a) */
  RT_EQUAL = 7, RT_NOT_EQUAL = 8, RT_GREATER = 9, RT_GREATER_EQUAL = 10, RT_LESS = 11, RT_LESS_EQUAL = 12, /* mod.rs:185-205 */
  RT_BINARY_COUNT = 13
};
rt_status rt_binary(rt_ctx* ctx, int op, const float* a, const int64_t* a_shape, int a_ndim,
                    const float* b, const int64_t* b_shape, int b_ndim, float* out);
rt_status rt_binary_backward(rt_ctx* ctx, int op, const float* a, const int64_t* a_shape, int a_ndim,
                             const float* b, const int64_t* b_shape, int b_ndim, const float* g,
                             float* da, float* db);
/* Sum `g` (shape g_shape) down to `target_shape`: leading extra dims and dims where the target
 * is 1 (unbroadcast, src/ops/cpu_backward.rs:523-678; Broadcast-op backward, src/tensor.rs:785-794). */
rt_status rt_unbroadcast(rt_ctx* ctx, const float* g, const int64_t* g_shape, int g_ndim,
                         const int64_t* target_shape, int t_ndim, float* out);
rt_status rt_broadcast_to(rt_ctx* ctx, const float* x, const int64_t* x_shape, int x_ndim,
                          const int64_t* out_shape, int out_ndim, float* out);     /* broadcast_to mod.rs:277 */
rt_status rt_transpose2d(rt_ctx* ctx, const float* x, int64_t rows, int64_t cols, float* out); /* transpose mod.rs:275 */
/* dst[starts + i] = src[i] for every index i of src (write a block into a larger tensor);
 * with it: slice_backward mod.rs:535 (= rt_fill 0 + assign), concat mod.rs:550. */
rt_status rt_slice_assign(rt_ctx* ctx, float* dst, const int64_t* dst_shape, int ndim, const int64_t* starts,
                          const float* src, const int64_t* src_shape);
/* out[i] = x[starts + i]: slice mod.rs:522, concat_backward mod.rs:563. */
rt_status rt_slice(rt_ctx* ctx, const float* x, const int64_t* x_shape, int ndim, const int64_t* starts,
                   const int64_t* out_shape, float* out);

/* out[i, :] = src[idx[i], :] (idx: n_idx int32 row numbers in DEVICE memory): the row gather of data::get_random_batch
 * (src/data.rs:125-209), done on the device instead of through a host copy of the whole data set. */
rt_status rt_gather_rows(rt_ctx* ctx, const float* src, int64_t rows, int64_t row_len, const int32_t* idx, int64_t n_idx, float* out);

/* out[c] += sum over r of x[r, c] for a row-major x[rows, cols]: the gradient of a bias that already holds a gradient (a bias
 * used at every timestep of a recurrent layer), accumulated in place in one launch.  Eight row lanes per column: meant for few rows. */
rt_status rt_sum_rows_accumulate(rt_ctx* ctx, const float* x, int64_t rows, int64_t cols, float* out);
/* ---- reductions over one axis of a tensor viewed as [outer, len, inner] ----------------------- */
enum {
  RT_RED_SUM = 0,       /* sum_along_axis mod.rs:291, sum_all mod.rs:293 */
  RT_RED_MEAN = 1,      /* mean mod.rs:298 */
  RT_RED_MAX = 2,       /* max mod.rs:160, max_along_axis mod.rs:295 */
  RT_RED_MIN = 3,       /* min mod.rs:164 */
  RT_RED_PROD = 4,      /* prod mod.rs:168 */
  RT_RED_LOGSUMEXP = 5, /* logsumexp mod.rs:173 */
  RT_RED_ARGMAX = 6,    /* argmax mod.rs:177 (index as f32, first maximum wins) */
  RT_RED_ARGMIN = 7,    /* argmin mod.rs:181 */
  RT_RED_COUNT = 8
};
rt_status rt_reduce(rt_ctx* ctx, int kind, const float* x, int64_t outer, int64_t len, int64_t inner, float* out);
/* dx[o,k,i] from g[o,i]:  SUM: g; MEAN: g/len; MAX/MIN: g * [|x - ext| < 1e-9] / (ties + 1e-9);
 * PROD: g * prod / (x + 1e-10); LOGSUMEXP: g * exp(x - lse).
 * sum_backward mod.rs:363, mean_backward mod.rs:339, max/min/prod/logsumexp_backward mod.rs:210-231. */
rt_status rt_reduce_backward(rt_ctx* ctx, int kind, const float* x, const float* g, int64_t outer, int64_t len,
                             int64_t inner, float* dx);
rt_status rt_sum_all_host(rt_ctx* ctx, const float* x, int64_t n, float* host_out); /* sum_all mod.rs:293; synchronises */
rt_status rt_log_softmax(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner, float* y); /* mod.rs:307 */
/* dx = g - exp(log_softmax(x)) * sum_axis(g)   (log_softmax_backward mod.rs:349) */
rt_status rt_log_softmax_backward(rt_ctx* ctx, const float* x, const float* g, int64_t outer, int64_t len,
                                  int64_t inner, float* dx);

/* Fused LSTM cell update (no counterpart in the reference, whose char-LSTM example builds the cell from slice, sigmoid, tanh,
 * mul and add ops: examples/lstm_char_rnn_cpu.rs).  gates is [batch, 4*hidden] with column blocks (input, forget, candidate,
 * output); c = sigmoid(f)*c_prev + sigmoid(i)*tanh(g); h = sigmoid(o)*tanh(c).  Each backward writes a full [batch, 4*hidden]
 * gradient for gates (zeros in the blocks it does not touch); gradient outputs may be NULL. */
rt_status rt_lstm_cell_c(rt_ctx* ctx, const float* gates, const float* c_prev, int64_t batch, int64_t hidden, float* c);
rt_status rt_lstm_cell_c_backward(rt_ctx* ctx, const float* gates, const float* c_prev, const float* dc, int64_t batch,
                                  int64_t hidden, float* dgates, float* dc_prev);
rt_status rt_lstm_cell_h(rt_ctx* ctx, const float* gates, const float* c, int64_t batch, int64_t hidden, float* h);
rt_status rt_lstm_cell_h_backward(rt_ctx* ctx, const float* gates, const float* c, const float* dh, int64_t batch,
                                  int64_t hidden, float* dgates, float* dc);

/* Fused classification loss (no counterpart in the reference, whose examples spell the chain out:
 * examples/train_mnist_cpu.rs:63-97): loss[0] = -(1/rows) * sum over rows and classes of targets * log_softmax(logits).
 * Backward: dlogits = -(g/rows) * (targets - softmax(logits) * sum_k targets), dtargets = -(g/rows) * log_softmax(logits);
 * g is the one-element upstream gradient on the device; either output may be NULL. */
rt_status rt_softmax_cross_entropy(rt_ctx* ctx, const float* logits, const float* targets, int64_t rows, int64_t classes,
                                   float* loss);
rt_status rt_softmax_cross_entropy_backward(rt_ctx* ctx, const float* logits, const float* targets, const float* g,
                                            int64_t rows, int64_t classes, float* dlogits, float* dtargets);

/* out[outer, inner] = sum over the middle axis of x[outer, len, inner], like rt_reduce(RT_RED_SUM), but the
 * call allocates nothing: the partial sums of a split reduction go to a fixed 1 MiB array in device memory
 * (one per device) instead of a block from the context's allocator.  No counterpart in the reference; it
 * serves callers that must not allocate while enqueueing (for example during stream capture).
 *  - A shape that needs more than 262144 partial sums, or outer > 65535 with inner > 1, returns
 *    RT_ERR_INVALID_OPERATION with a message; use rt_reduce for those.
 *  - The first call on a device looks up the array's address (cudaGetSymbolAddress), which may load the
 *    module: make one call (any shape, outer = 0 is enough) before starting a stream capture.
 *  - Calls that overlap on one device (other streams or contexts) share the array and race; calls on one
 *    stream are ordered. */
rt_status rt_reduce_sum_static_scratch(rt_ctx* ctx, const float* x, int64_t outer, int64_t len, int64_t inner,
                                       float* out);

/* ---- pooling (max_pool2d mod.rs:144, max_pool2d_backward mod.rs:151) -------------------------
 * idx holds the in-window position ky*kw+kx of the first maximum as f32 (strict >, padding = -inf). */
rt_status rt_max_pool2d(rt_ctx* ctx, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, int kh, int kw,
                        int sh, int sw, int ph, int pw, float* y, float* idx);
rt_status rt_max_pool2d_backward(rt_ctx* ctx, const float* g, const float* idx, int64_t n, int64_t c, int64_t h,
                                 int64_t w, int kh, int kw, int sh, int sw, int ph, int pw, float* dx);
/* Fused relu + max_pool2d (no counterpart in the reference, whose models call relu and max_pool2d one after the other,
 * e.g. examples/train_mnist_cnn_cpu.rs): y, idx = max_pool2d(relu(x)) without materialising relu(x); the backward routes g
 * through idx and masks it with x > 0 in the same pass.  Values and indices are bit-identical to the two separate ops. */
rt_status rt_relu_max_pool2d(rt_ctx* ctx, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, int kh, int kw,
                             int sh, int sw, int ph, int pw, float* y, float* idx);
rt_status rt_relu_max_pool2d_backward(rt_ctx* ctx, const float* x, const float* g, const float* idx, int64_t n, int64_t c,
                                      int64_t h, int64_t w, int kh, int kw, int sh, int sw, int ph, int pw, float* dx);
/* The same from the POOLED output, for a 2x2 window with stride 2 over an un-pooled tensor [n, c, h, w] with even h and w:
 * dx routes g through idx where y > 0 (y = relu of the window's maximum, so y > 0 exactly when the input at the saved position
 * was positive).  Bit-identical to rt_relu_max_pool2d_backward; the un-pooled tensor is not needed. */
rt_status rt_relu_max_pool2x2_backward_from_output(rt_ctx* ctx, const float* y, const float* g, const float* idx, int64_t n, int64_t c,
                                                   int64_t h, int64_t w, float* dx);

/* ---- dense contractions ---------------------------------------------------------------------- */
/* C[M,N] = op(A) * op(B) (+ C when accumulate != 0); row-major with leading dimensions.
 * trans_a: A is stored [K,M]; trans_b: B is stored [N,K].  matmul mod.rs:93 and the
 * transposed products of its backward closure (src/ops/mod.rs:161-175), without materialising
 * the transposes. */
rt_status rt_gemm(rt_ctx* ctx, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k, const float* a,
                  int64_t lda, const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate);
/* da[M,K] = g * b^T, db[K,N] = a^T * g   (matmul_backward mod.rs:324); NULL skips one. */
rt_status rt_matmul_backward(rt_ctx* ctx, const float* a, const float* b, const float* g, int64_t m, int64_t k,
                             int64_t n, float* da, float* db);
/* The same with db_sum[K,N] += a^T * g: for a weight that already holds a gradient (used at every timestep of a recurrent
 * layer), the product accumulates into it instead of a product followed by an addition (what add_grad does, src/tensor.rs:1099). */
rt_status rt_matmul_backward_accumulate(rt_ctx* ctx, const float* a, const float* b, const float* g, int64_t m, int64_t k,
                                        int64_t n, float* da, float* db_sum);
/* conv2d mod.rs:101: x[N,Cin,H,W], w[Cout,Cin,kh,kw], bias[Cout] or NULL -> y[N,Cout,Ho,Wo] */
rt_status rt_conv2d(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n, int64_t cin,
                    int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw, float* y);
/* Fused conv2d + bias + relu + max_pool2d(2x2, stride 2) (no counterpart in the reference, whose CNN example calls the three
 * ops one after the other, examples/train_mnist_cnn_cpu.rs:216-233): y, idx [n, cout, Ho/2, Wo/2]; the convolution output (Ho x
 * Wo, both even) is not kept.  Values and indices are bit-identical to rt_conv2d -> relu -> rt_max_pool2d.  Single-channel 3x3
 * unit-stride layers run as one kernel; other shapes as the convolution into scratch memory followed by the fused relu + pool
 * kernel.  Backward: rt_relu_max_pool2x2_backward_from_output, then rt_conv2d_backward. */
rt_status rt_conv2d_relu_max_pool2x2(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n, int64_t cin, int64_t h,
                                     int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw, float* y, float* idx);
/* conv2d_backward mod.rs:111: any of dx, dw, db may be NULL.  dx is the mathematically correct
 * input gradient (the reference CPU code's col2im reuses column 0, src/ops/cpu_ops.rs:266). */
rt_status rt_conv2d_backward(rt_ctx* ctx, const float* x, const float* w, const float* g, int64_t n, int64_t cin,
                             int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw, int ph, int pw,
                             float* dx, float* dw, float* db);
/* conv2d_transpose mod.rs:125: x[N,Cin,H,W], w[Cin,Cout,kh,kw] -> y[N,Cout,(H-1)sh+kh-2ph,(W-1)sw+kw-2pw] */
rt_status rt_conv2d_transpose(rt_ctx* ctx, const float* x, const float* w, const float* bias, int64_t n,
                              int64_t cin, int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh, int sw,
                              int ph, int pw, float* y);
/* conv2d_transpose_backward mod.rs:135; g is [N,Cout,OH,OW]. */
rt_status rt_conv2d_transpose_backward(rt_ctx* ctx, const float* x, const float* w, const float* g, int64_t n,
                                       int64_t cin, int64_t h, int64_t wd, int64_t cout, int kh, int kw, int sh,
                                       int sw, int ph, int pw, float* dx, float* dw, float* db);

/* ---- optimizer steps (in place) ---------------------------------------------------------------- */
rt_status rt_sgd_step(rt_ctx* ctx, float* param, const float* grad, int64_t n, float lr);            /* mod.rs:256 */
rt_status rt_momentum_sgd_step(rt_ctx* ctx, float* param, const float* grad, float* velocity, int64_t n,
                               float lr, float momentum);                                              /* mod.rs:18 */
rt_status rt_adagrad_step(rt_ctx* ctx, float* param, const float* grad, float* accum, int64_t n, float lr,
                          float epsilon);                                                              /* mod.rs:30 */
rt_status rt_adam_step(rt_ctx* ctx, float* param, const float* grad, float* m, float* v, int64_t n, float lr,
                       float beta1, float beta2, float epsilon, int64_t t);                           /* mod.rs:262 */
/* One launch over a list of tensors (the whole model): kind 0 sgd, 1 adam, 2 momentum, 3 adagrad.
 * The gradient is first multiplied by grad_scale (1/world after an all-reduce) and, when
 * clip != 0, clamped to [clip_lo, clip_hi] BEFORE the scale (Backend::clip, mod.rs:629).
 * state2 is only read for Adam.  Pointer arrays are host arrays of device pointers. */
rt_status rt_optimizer_step_multi(rt_ctx* ctx, int kind, int n_tensors, float* const* params,
                                  const float* const* grads, float* const* state1, float* const* state2,
                                  const int64_t* sizes, float lr, float beta1, float beta2, float epsilon,
                                  float momentum, int64_t t, float grad_scale, int clip, float clip_lo,
                                  float clip_hi);

/* ---- data-parallel gradient exchange (no counterpart in the reference: it has no distributed code) */
/* Copies a list of gradient tensors into one flat buffer (optionally clamping), so that one
 * all-reduce covers the model. */
rt_status rt_pack_flat(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat,
                       int clip, float clip_lo, float clip_hi);
#define RT_DP_ID_BYTES 128
rt_status rt_dp_unique_id(uint8_t id[RT_DP_ID_BYTES]);                /* rank 0 creates, every rank receives a copy */
/* Joins the communicator.  rt_dp_init_deadline with timeout_ms > 0 creates it in NCCL's non-blocking mode and polls
 * ncclCommGetAsyncError until every rank has joined or the deadline has passed: a rank that never joins ends the call with
 * RT_ERR_TIMEOUT (the half-built communicator is aborted and the context stays usable) instead of blocking for ever.  The
 * same deadline then bounds every later wait of this context on the communicator (rt_dp_allreduce_sum's enqueue,
 * rt_dp_wait_event).  timeout_ms <= 0, or an NCCL without the non-blocking API: the plain blocking ncclCommInitRank.
 * rt_dp_init joins a BLOCKING communicator (on a non-blocking one every all-reduce has to be polled, which costs the host
 * more than 0.1 ms per step) unless RT_B200_NCCL_NONBLOCKING=1 is set (deadline RT_B200_DP_TIMEOUT_MS, default 120000); make
 * sure beforehand, on the host, that every rank is there (rusttensor_b200/dp_setup.py does that with a deadline). */
rt_status rt_dp_init(rt_ctx* ctx, int rank, int world, const uint8_t id[RT_DP_ID_BYTES]);
rt_status rt_dp_init_deadline(rt_ctx* ctx, int rank, int world, const uint8_t id[RT_DP_ID_BYTES], int64_t timeout_ms);
rt_status rt_dp_allreduce_sum(rt_ctx* ctx, float* buf, int64_t n);    /* in place, on the context's stream */
/* One poll of ncclCommGetAsyncError: RT_OK while the communicator is healthy (or there is none); an asynchronous error
 * (a peer that died, a failed transport) aborts the communicator and returns RT_ERR_NCCL; *nccl_code gets NCCL's code. */
rt_status rt_dp_async_error(rt_ctx* ctx, int* nccl_code);
/* Waits for an event recorded behind a step like rt_event_synchronize, but as a watchdog: the host polls the event and
 * the communicator's asynchronous error together; on an error, or when the context's deadline passes first, the
 * communicator is aborted (which ends a collective kernel stuck on a missing peer) and RT_ERR_NCCL / RT_ERR_TIMEOUT is
 * returned.  Without a communicator it is rt_event_synchronize. */
rt_status rt_dp_wait_event(rt_ctx* ctx, rt_event* ev);
rt_status rt_dp_finalize(rt_ctx* ctx);

/* ---- gradient exchange fused into the optimizer step over peer memory (new) ----------------------------------
 * Instead of all-reducing the flat gradient buffer and then running the optimizer, every rank reads the other ranks'
 * flat buffers directly over NVLink (plain peer loads) inside the optimizer kernel, adds them in rank order (the same
 * order on every rank, so all ranks compute bit-identical sums) and applies the update: one kernel does the exchange
 * and the step.  Set-up: each rank exports its buffers with rt_ipc_export, the 64-byte handles travel between the
 * processes by any means, and each rank opens the others' with rt_ipc_open.
 * Per step: rt_dp_step_begin, (forward, backward), rt_pack_flat_alternating into flat[step & 1], rt_dp_signal_peers (writes
 * the step number into slot `rank` of every peer's flag array once the pack has finished), rt_dp_wait_peers (one block
 * waits, with a bounded number of polls, until every peer has signalled the step), rt_optimizer_step_multi_peers.  All of
 * them take their step number from device memory, so the sequence can be captured once and replayed as one CUDA graph.
 * Two flat buffers alternate: a rank can only overwrite flat[s & 1] at step s+2, after every peer has signalled step s+1
 * and has therefore finished reading it. */
#define RT_IPC_HANDLE_BYTES 64
#define RT_DP_MAX_PEERS 8
rt_status rt_ipc_export(rt_ctx* ctx, void* device_ptr, uint8_t handle[RT_IPC_HANDLE_BYTES]); /* ptr: start of an rt_malloc block */
rt_status rt_ipc_open(rt_ctx* ctx, const uint8_t handle[RT_IPC_HANDLE_BYTES], void** peer_ptr);
rt_status rt_ipc_close(rt_ctx* ctx, void* peer_ptr);
/* Step state in device memory: RT_STEP_STATE_WORDS ints, zero before the first step.  word 0 = exchange step number,
 * word 1 = step for which the peers' gradients are complete (negative: the wait for that step ran out), word 2 = optimizer
 * step count t, word 3 = time this rank has spent in rt_dp_wait_peers so far, in units of 64 ns (a diagnostic).  Keeping it on the device lets a whole training step - including the exchange and Adam's bias
 * corrections - be replayed from one CUDA graph.  rt_dp_step_begin adds one to words 0 and 2. */
#define RT_STEP_STATE_WORDS 4
rt_status rt_dp_step_begin(rt_ctx* ctx, int* step_state);
/* rt_optimizer_step_multi with t read from step_state (word 2) on the device. */
rt_status rt_optimizer_step_multi_device_t(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                                           float* const* state1, float* const* state2, const int64_t* sizes, float lr, float beta1,
                                           float beta2, float epsilon, float momentum, const int* step_state, float grad_scale,
                                           int clip, float clip_lo, float clip_hi);
/* rt_pack_flat into flat0 or flat1, whichever the step number selects (buffer = step & 1). */
rt_status rt_pack_flat_alternating(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat0,
                                   float* flat1, const int* step_state, int clip, float clip_lo, float clip_hi);
/* rt_pack_flat_alternating and rt_dp_signal_peers in one launch: the block of the pack kernel that finishes last writes the
 * flags.  Falls back to the two launches when the tensor list needs more than one pack launch. */
rt_status rt_pack_flat_signal(rt_ctx* ctx, int n_tensors, const float* const* srcs, const int64_t* sizes, float* flat0, float* flat1,
                              const int* step_state, int clip, float clip_lo, float clip_hi, int* const* peer_flags, int rank,
                              int world);
/* peer_flags[r] = rank r's flag array (world ints) as opened on this rank; the entry of this rank is ignored.  Writes the
 * current step number into slot `rank` of every peer's array, after everything queued before it on the stream. */
rt_status rt_dp_signal_peers(rt_ctx* ctx, int* const* peer_flags, int rank, int world, const int* step_state);
/* One block waits until every peer has signalled the current step (local_flags = this rank's flag array) and marks the
 * step ready in step_state; after spin_limit polls per peer (0 = default, about ten seconds) it gives up: the step is marked
 * failed, a code (16 + the silent rank) goes to the status word, and rt_optimizer_step_multi_peers for this step changes
 * nothing - in none of its blocks.  The next synchronising call returns RT_ERR_TIMEOUT. */
rt_status rt_dp_wait_peers(rt_ctx* ctx, const int* local_flags, int rank, int world, int* step_state, uint32_t spin_limit);
/* Like rt_optimizer_step_multi_device_t, with the gradient of every element read from all ranks: grads[i] points into THIS
 * rank's flats0[rank]; the same offsets are read from every flats0[r] (odd steps: flats1[r]) and added in rank order.
 * grad_scale is normally 1/world.  Runs only if rt_dp_wait_peers marked the step ready. */
rt_status rt_optimizer_step_multi_peers(rt_ctx* ctx, int kind, int n_tensors, float* const* params, const float* const* grads,
                                        float* const* state1, float* const* state2, const int64_t* sizes, float lr, float beta1,
                                        float beta2, float epsilon, float momentum, float grad_scale, const float* const* flats0,
                                        const float* const* flats1, int rank, int world, const int* step_state);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
