// The five benchmark workloads written once against the generic op front-end,
// the way the reference's examples are written against `Backend`:
//   C1  MLP            examples/train_mnist_cpu.rs:46-97 (+ biases as examples/sine_regression_cpu.rs:41-43)
//   C2  elementwise / reduction chain with a broadcast bias (microbenchmark graph)
//   C3  CNN            examples/train_mnist_cnn_cpu.rs:189-233 (3x3 kernels, 32/64 channels)
//   C4  conv -> relu -> pool -> conv-transpose -> mse
//   C5  character LSTM examples/lstm_char_rnn_cpu.rs:98-138, 405-435 (fused gate matrix)
// The same templates are instantiated for the CUDA backend (the product) and,
// in the test-only oracle build, for the CPU restatement.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "autograd.hpp"

namespace rt {
namespace models {

enum Config { C1_MLP = 1, C2_ELEMENTWISE = 2, C3_CNN = 3, C4_CONV_CONVT = 4, C5_LSTM = 5 };

template <class B>
struct Workload {
  int config = 0;
  std::vector<size_t> dims;              // configuration-specific sizes (see make_workload)
  std::vector<Tensor<B>> params;         // tensors that receive gradients, in optimizer order
  std::vector<std::string> names;
  std::vector<Shape> input_shapes;       // shapes of the per-step inputs
  // optimizer: 0 none, 1 Adam, 2 MomentumSGD
  int optimizer = 0;
  float lr = 1e-3f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, momentum = 0.9f;
  bool clip_grads = false;
  float clip_lo = -5.f, clip_hi = 5.f;
  // true: relu + max_pool2d and the classification loss go through the fused ops (ops::fused_*); same mathematics
  bool fused_forward = false;

  void add_param(const std::string& n, const Shape& s) {
    params.push_back(Tensor<B>::zeros(s, true));
    names.push_back(n);
  }
};

// dims:
//  C1: {batch, in, hidden, classes}            inputs: X[batch,in], Y[batch,classes]
//  C2: {rows, cols}                            inputs: none (X and b are the "params")
//  C3: {batch, hw, c1, c2, fc, classes}        inputs: X[batch,1,hw,hw], Y[batch,classes]
//  C4: {batch, cin, hw, cmid}                  inputs: X[batch,cin,hw,hw] (requires grad), T same shape
//  C5: {vocab, hidden, seq, batch}             inputs: X[seq*batch, vocab] one-hot, Y likewise (time-major)
template <class B>
Workload<B> make_workload(int config, const std::vector<size_t>& d) {
  Workload<B> w;
  if (config >= 100) {  // 100 + c: configuration c built from the fused forward ops
    config -= 100;
    w.fused_forward = true;
  }
  w.config = config;
  w.dims = d;
  auto need = [&](size_t n) {
    if (d.size() != n) throw Error::invalid_op("make_workload: wrong number of dims for config");
  };
  switch (config) {
    case C1_MLP:
      need(4);
      w.add_param("w1", {d[1], d[2]});
      w.add_param("b1", {d[2]});
      w.add_param("w2", {d[2], d[3]});
      w.add_param("b2", {d[3]});
      w.input_shapes = {{d[0], d[1]}, {d[0], d[3]}};
      w.optimizer = 1;
      break;
    case C2_ELEMENTWISE:
      need(2);
      w.add_param("x", {d[0], d[1]});
      w.add_param("b", {d[1]});
      w.optimizer = 0;
      break;
    case C3_CNN: {
      need(6);
      size_t hw = d[1], p2 = hw / 4;
      w.add_param("conv1_w", {d[2], 1, 3, 3});
      w.add_param("conv1_b", {d[2]});
      w.add_param("conv2_w", {d[3], d[2], 3, 3});
      w.add_param("conv2_b", {d[3]});
      w.add_param("fc1_w", {d[3] * p2 * p2, d[4]});
      w.add_param("fc1_b", {d[4]});
      w.add_param("fc2_w", {d[4], d[5]});
      w.add_param("fc2_b", {d[5]});
      w.input_shapes = {{d[0], 1, hw, hw}, {d[0], d[5]}};
      w.optimizer = 1;
      break;
    }
    case C4_CONV_CONVT:
      need(4);
      w.add_param("conv_w", {d[3], d[1], 3, 3});
      w.add_param("conv_b", {d[3]});
      w.add_param("convt_w", {d[3], d[1], 4, 4});  // [Cin_T, Cout_T, kh, kw]
      w.add_param("convt_b", {d[1]});
      w.input_shapes = {{d[0], d[1], d[2], d[2]}, {d[0], d[1], d[2], d[2]}};
      w.optimizer = 2;
      w.lr = 1e-2f;
      w.momentum = 0.9f;
      break;
    case C5_LSTM:
      need(4);
      w.add_param("w_gates", {d[0] + d[1], 4 * d[1]});  // [x,h] -> i,f,g,o column blocks
      w.add_param("b_gates", {4 * d[1]});
      w.add_param("why", {d[1], d[0]});
      w.add_param("by", {d[0]});
      w.input_shapes = {{d[2] * d[3], d[0]}, {d[2] * d[3], d[0]}};
      w.optimizer = 1;
      w.clip_grads = true;
      break;
    default:
      throw Error::invalid_op("make_workload: unknown config");
  }
  return w;
}

// -loss = mean over the batch of sum_k y*log_softmax (examples/train_mnist_cpu.rs:63-97)
template <class B>
Tensor<B> nll_loss(const Tensor<B>& log_probs, const Tensor<B>& y) {
  Tensor<B> e = ops::mul(log_probs, y);
  Tensor<B> per = ops::sum(e, 1);
  Tensor<B> m = ops::mean(per, std::nullopt);
  Tensor<B> minus_one = Tensor<B>::from_vec({-1.0f}, Shape{}, false);
  return ops::mul(m, minus_one);
}

// x·w + b as the examples write it: the bias is broadcast to [batch, out] by its own op and then added.  With
// `direct_bias` the add broadcasts the bias itself (operator broadcasting, src/ops/mod.rs add), one kernel fewer.
template <class B>
Tensor<B> linear(const Tensor<B>& x, const Tensor<B>& w, const Tensor<B>& b, bool direct_bias = false) {
  Tensor<B> h = ops::matmul(x, w);
  if (direct_bias) return ops::add(h, b);
  return ops::add(h, b.broadcast_to({x.shape()[0], w.shape()[1]}));
}

// Builds the forward graph of one step and returns the scalar loss.  `inputs`
// follow Workload::input_shapes; C4's first input must have been created with
// requires_grad = true by the caller when its gradient is wanted.
template <class B>
Tensor<B> forward_loss(const Workload<B>& w, const std::vector<Tensor<B>>& in) {
  const auto& p = w.params;
  const auto& d = w.dims;
  const Pair two{2, 2}, zero{0, 0};
  auto relu_pool = [&](const Tensor<B>& x) {
    return w.fused_forward ? ops::fused_relu_max_pool2d(x, two, two, zero) : ops::max_pool2d(ops::relu(x), two, two, zero);
  };
  switch (w.config) {
    case C1_MLP: {
      Tensor<B> h = ops::relu(linear(in.at(0), p[0], p[1], w.fused_forward));
      Tensor<B> logits = linear(h, p[2], p[3], w.fused_forward);
      if (w.fused_forward) return ops::fused_softmax_nll(logits, in.at(1));
      return nll_loss(ops::log_softmax(logits, 1), in.at(1));
    }
    case C2_ELEMENTWISE: {
      const Tensor<B>&x = p[0], &b = p[1];
      Tensor<B> t1 = ops::mul(x, b);
      Tensor<B> t2 = ops::tanh(t1);
      Tensor<B> t3 = ops::square(x);
      Tensor<B> t4 = ops::mul_scalar(t3, -1.0f);
      Tensor<B> t5 = ops::exp(t4);
      Tensor<B> t6 = ops::sin(x);
      Tensor<B> one = Tensor<B>::from_vec({1.0f}, Shape{}, false);
      Tensor<B> t7 = ops::add(t3, one);
      Tensor<B> t8 = ops::div(t6, t7);
      Tensor<B> y = ops::add(ops::add(t2, t5), t8);
      Tensor<B> l = ops::logsumexp(y, 1);
      return ops::sum(l, std::nullopt);
    }
    case C3_CNN: {
      size_t n = in.at(0).shape()[0];
      auto block = [&](const Tensor<B>& x, const Tensor<B>& wt, const Tensor<B>& b) {
        if (w.fused_forward) return ops::fused_conv2d_relu_max_pool2d(x, wt, &b, {1, 1}, {1, 1});
        return relu_pool(ops::conv2d(x, wt, &b, {1, 1}, {1, 1}));
      };
      Tensor<B> p1 = block(in[0], p[0], p[1]);
      Tensor<B> p2 = block(p1, p[2], p[3]);
      Tensor<B> flat = p2.view({n, p[4].shape()[0]});
      Tensor<B> f1 = ops::relu(linear(flat, p[4], p[5], w.fused_forward));
      Tensor<B> logits = linear(f1, p[6], p[7], w.fused_forward);
      if (w.fused_forward) return ops::fused_softmax_nll(logits, in.at(1));
      return ops::softmax_cross_entropy(logits, in.at(1), 1, Reduction::Mean);
    }
    case C4_CONV_CONVT: {
      Tensor<B> pl = w.fused_forward ? ops::fused_conv2d_relu_max_pool2d(in.at(0), p[0], &p[1], {1, 1}, {1, 1})
                                     : relu_pool(ops::conv2d(in.at(0), p[0], &p[1], {1, 1}, {1, 1}));
      Tensor<B> up = ops::conv2d_transpose(pl, p[2], &p[3], {2, 2}, {1, 1});
      return ops::mse_loss(up, in.at(1), Reduction::Mean);
    }
    case C5_LSTM: {
      size_t V = d[0], H = d[1], T = d[2], Bn = d[3];
      Tensor<B> h = Tensor<B>::zeros({Bn, H}, false), c = Tensor<B>::zeros({Bn, H}, false);
      Tensor<B> total;
      std::vector<Tensor<B>> hs;  // fused variant: the hidden states of all timesteps, for ONE output projection
      for (size_t t = 0; t < T; ++t) {
        Tensor<B> xh = w.fused_forward ? ops::fused_rows_concat(in.at(0), t * Bn, (t + 1) * Bn, h)
                                       : ops::concat<B>({ops::slice(in.at(0), {{t * Bn, (t + 1) * Bn}, {0, V}}), h}, 1);
        Tensor<B> gates = linear(xh, p[0], p[1], w.fused_forward);
        if (w.fused_forward) {
          c = ops::fused_lstm_cell_c(gates, c);
          h = ops::fused_lstm_cell_h(gates, c);
          hs.push_back(h);
          continue;
        }
        Tensor<B> y_t = ops::slice(in.at(1), {{t * Bn, (t + 1) * Bn}, {0, V}});
        Tensor<B> ig = ops::sigmoid(ops::slice(gates, {{0, Bn}, {0, H}}));
        Tensor<B> fg = ops::sigmoid(ops::slice(gates, {{0, Bn}, {H, 2 * H}}));
        Tensor<B> gg = ops::tanh(ops::slice(gates, {{0, Bn}, {2 * H, 3 * H}}));
        Tensor<B> og = ops::sigmoid(ops::slice(gates, {{0, Bn}, {3 * H, 4 * H}}));
        c = ops::add(ops::mul(fg, c), ops::mul(ig, gg));
        h = ops::mul(og, ops::tanh(c));
        Tensor<B> logits = linear(h, p[2], p[3], false);
        Tensor<B> l = ops::softmax_cross_entropy(logits, y_t, 1, Reduction::Mean);
        total = t == 0 ? l : ops::add(total, l);
      }
      if (w.fused_forward) {
        // The example projects and scores every timestep on its own (examples/lstm_char_rnn_cpu.rs:405-435) and adds the T mean
        // losses.  The targets are already time-major [T*B, V], so one [T*B, H] x [H, V] product and one loss over all rows
        // give the same sum: sum_t mean_b l(t, b) = T * mean over all T*B rows.
        Tensor<B> all_h = ops::concat<B>(hs, 0);
        Tensor<B> logits = linear(all_h, p[2], p[3], true);
        total = ops::mul_scalar(ops::fused_softmax_nll(logits, in.at(1)), (float)T);
      }
      return total;
    }
    default:
      throw Error::invalid_op("forward_loss: unknown config");
  }
}

// One optimisation step with the reference's per-tensor optimizer API
// (examples/train_mnist_cnn_cpu.rs:138-156): zero_grad, forward, backward,
// optional gradient clip through B::clip, optimizer step.
template <class B>
struct Trainer {
  Workload<B> w;
  std::unique_ptr<optim::Adam<B>> adam;
  std::unique_ptr<optim::MomentumSGD<B>> msgd;

  explicit Trainer(Workload<B> wl) : w(std::move(wl)) {}
  void ensure_optimizer() {
    if (w.optimizer == 1 && !adam) adam.reset(new optim::Adam<B>(w.params, w.lr, w.beta1, w.beta2, w.eps));
    if (w.optimizer == 2 && !msgd) msgd.reset(new optim::MomentumSGD<B>(w.params, w.lr, w.momentum));
  }
  Tensor<B> forward_backward(const std::vector<Tensor<B>>& in) {
    for (auto& p : w.params) p.zero_grad();
    Tensor<B> loss = forward_loss(w, in);
    loss.backward();
    if (w.clip_grads)
      for (auto& p : w.params)
        if (p.grad()) p.set_grad(B::clip(*p.grad(), w.clip_lo, w.clip_hi));
    return loss;
  }
  void optimizer_step() {
    ensure_optimizer();
    if (adam) adam->step();
    if (msgd) msgd->step();
  }
  Tensor<B> step(const std::vector<Tensor<B>>& in) {
    Tensor<B> loss = forward_backward(in);
    optimizer_step();
    return loss;
  }
};

}  // namespace models
}  // namespace rt
