// Fused LSTM cell update (no counterpart in the reference, whose char-LSTM example builds the cell from slice,
// sigmoid, tanh, mul and add ops: examples/lstm_char_rnn_cpu.rs).  gates is [B, 4H] with the column blocks
// (input, forget, candidate, output) = [0,H), [H,2H), [2H,3H), [3H,4H):
//   c = sigmoid(f) * c_prev + sigmoid(i) * tanh(g)           rt_lstm_cell_c
//   h = sigmoid(o) * tanh(c)                                   rt_lstm_cell_h
// Two single-output ops, so that each fits the one-output Op of the autograd graph; each backward writes a full [B,4H]
// gradient for gates (zeros in the blocks it does not touch) and the two are added by the graph's accumulation.
// Derivatives are written like the reference's backward functions: sigmoid' = s(1-s), tanh' = 1 - t^2.
#include "rt_internal.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(kThreads) lstm_c_fwd(const float* __restrict__ gates, const float* __restrict__ c_prev,
                                                       float* __restrict__ c, int64_t n, int H) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = e / H;
    const int j = (int)(e - b * H);
    const float* g = gates + b * 4 * H;
    c[e] = sigmoidf_(__ldg(g + H + j)) * __ldg(c_prev + e) + sigmoidf_(__ldg(g + j)) * tanhf(__ldg(g + 2 * H + j));
  }
}

__global__ void __launch_bounds__(kThreads) lstm_c_bwd(const float* __restrict__ gates, const float* __restrict__ c_prev,
                                                       const float* __restrict__ dc, float* __restrict__ dgates,
                                                       float* __restrict__ dc_prev, int64_t n, int H) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = e / H;
    const int j = (int)(e - b * H);
    const float* g = gates + b * 4 * H;
    const float si = sigmoidf_(__ldg(g + j)), sf = sigmoidf_(__ldg(g + H + j)), tg = tanhf(__ldg(g + 2 * H + j));
    const float d = __ldg(dc + e);
    if (dgates) {
      float* dg = dgates + b * 4 * H;
      dg[j] = (d * tg) * si * (1.0f - si);
      dg[H + j] = (d * __ldg(c_prev + e)) * sf * (1.0f - sf);
      dg[2 * H + j] = (d * si) * (1.0f - tg * tg);
      dg[3 * H + j] = 0.f;
    }
    if (dc_prev) dc_prev[e] = d * sf;
  }
}

__global__ void __launch_bounds__(kThreads) lstm_h_fwd(const float* __restrict__ gates, const float* __restrict__ c,
                                                       float* __restrict__ h, int64_t n, int H) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = e / H;
    const int j = (int)(e - b * H);
    h[e] = sigmoidf_(__ldg(gates + b * 4 * H + 3 * H + j)) * tanhf(__ldg(c + e));
  }
}

__global__ void __launch_bounds__(kThreads) lstm_h_bwd(const float* __restrict__ gates, const float* __restrict__ c,
                                                       const float* __restrict__ dh, float* __restrict__ dgates,
                                                       float* __restrict__ dc, int64_t n, int H) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = e / H;
    const int j = (int)(e - b * H);
    const float so = sigmoidf_(__ldg(gates + b * 4 * H + 3 * H + j)), tc = tanhf(__ldg(c + e));
    const float d = __ldg(dh + e);
    if (dgates) {
      float* dg = dgates + b * 4 * H;
      dg[j] = 0.f;
      dg[H + j] = 0.f;
      dg[2 * H + j] = 0.f;
      dg[3 * H + j] = (d * tc) * so * (1.0f - so);
    }
    if (dc) dc[e] = (d * so) * (1.0f - tc * tc);
  }
}

rt_status check_dims(rt_ctx* ctx, int64_t batch, int64_t hidden, const char* who) {
  if (batch < 0 || hidden < 0) RT_FAIL(ctx, RT_ERR_INVALID_INDEX, "%s: negative extent", who);
  if (hidden >= (1 << 28)) RT_FAIL(ctx, RT_ERR_INVALID_OPERATION, "%s: hidden size too large", who);
  return RT_OK;
}

}  // namespace

extern "C" {

rt_status rt_lstm_cell_c(rt_ctx* ctx, const float* gates, const float* c_prev, int64_t batch, int64_t hidden, float* c) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_dims(ctx, batch, hidden, "rt_lstm_cell_c");
  if (st != RT_OK) return st;
  const int64_t n = batch * hidden;
  if (n == 0) return RT_OK;
  RT_CHECK_PTR(ctx, gates);
  RT_CHECK_PTR(ctx, c_prev);
  RT_CHECK_PTR(ctx, c);
  lstm_c_fwd<<<rt_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(gates, c_prev, c, n, (int)hidden);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_lstm_cell_c_backward(rt_ctx* ctx, const float* gates, const float* c_prev, const float* dc, int64_t batch,
                                  int64_t hidden, float* dgates, float* dc_prev) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_dims(ctx, batch, hidden, "rt_lstm_cell_c_backward");
  if (st != RT_OK) return st;
  const int64_t n = batch * hidden;
  if (n == 0 || (!dgates && !dc_prev)) return RT_OK;
  RT_CHECK_PTR(ctx, gates);
  RT_CHECK_PTR(ctx, c_prev);
  RT_CHECK_PTR(ctx, dc);
  lstm_c_bwd<<<rt_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(gates, c_prev, dc, dgates, dc_prev, n, (int)hidden);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_lstm_cell_h(rt_ctx* ctx, const float* gates, const float* c, int64_t batch, int64_t hidden, float* h) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_dims(ctx, batch, hidden, "rt_lstm_cell_h");
  if (st != RT_OK) return st;
  const int64_t n = batch * hidden;
  if (n == 0) return RT_OK;
  RT_CHECK_PTR(ctx, gates);
  RT_CHECK_PTR(ctx, c);
  RT_CHECK_PTR(ctx, h);
  lstm_h_fwd<<<rt_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(gates, c, h, n, (int)hidden);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

rt_status rt_lstm_cell_h_backward(rt_ctx* ctx, const float* gates, const float* c, const float* dh, int64_t batch,
                                  int64_t hidden, float* dgates, float* dc) {
  RT_CHECK_CTX(ctx);
  rt_status st = check_dims(ctx, batch, hidden, "rt_lstm_cell_h_backward");
  if (st != RT_OK) return st;
  const int64_t n = batch * hidden;
  if (n == 0 || (!dgates && !dc)) return RT_OK;
  RT_CHECK_PTR(ctx, gates);
  RT_CHECK_PTR(ctx, c);
  RT_CHECK_PTR(ctx, dh);
  lstm_h_bwd<<<rt_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(gates, c, dh, dgates, dc, n, (int)hidden);
  RT_LAUNCHED(ctx);
  return RT_OK;
}

}  // extern "C"
