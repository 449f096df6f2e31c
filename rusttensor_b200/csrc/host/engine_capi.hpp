// A plain-C view of the generic autograd engine, so that a scripting host (the
// Python tests and the benchmark driver) can build the same graphs a Rust user
// builds with `ops::*`, call `backward()` and run optimizer steps.
//
// RT_DEFINE_ENGINE_CAPI(prefix, Backend) emits `extern "C"` functions named
// `<prefix>_*` for one backend.  The shipped library instantiates it for the
// CUDA backend; the test-only oracle build instantiates it for its CPU
// restatement, which is what makes differential tests symmetric (the reference
// does the same with Tensor<CpuBackend> vs Tensor<CudaBackend>,
// tests/ops_cuda_backward_tests.rs:74-144).
//
// Every function returns 0 on success or the numeric value of rt::ErrorKind;
// `<prefix>_last_error()` returns the message of the last failure.
#pragma once
#include <cstring>
#include <map>
#include <string>

#include "autograd.hpp"
#include "models.hpp"

namespace rt {
namespace capi {

template <class B>
struct Registry {
  std::map<int64_t, Tensor<B>> tensors;
  std::map<int64_t, std::shared_ptr<models::Trainer<B>>> trainers;
  struct Optim {
    int kind;  // 0 sgd 1 adam 2 momentum 3 adagrad
    std::shared_ptr<optim::Sgd<B>> sgd;
    std::shared_ptr<optim::Adam<B>> adam;
    std::shared_ptr<optim::MomentumSGD<B>> mom;
    std::shared_ptr<optim::AdaGrad<B>> ada;
  };
  std::map<int64_t, Optim> optims;
  int64_t next = 1;
  std::string last_error;
  int64_t put(Tensor<B> t) {
    tensors[next] = std::move(t);
    return next++;
  }
  Tensor<B>& get(int64_t h) {
    auto it = tensors.find(h);
    if (it == tensors.end()) throw Error::invalid_op("unknown tensor handle " + std::to_string(h));
    return it->second;
  }
  static Registry& instance() {
    static Registry r;
    return r;
  }
};

inline Shape to_shape(const int64_t* s, int nd) {
  Shape r(nd);
  for (int i = 0; i < nd; ++i) r[i] = (size_t)s[i];
  return r;
}
inline std::optional<size_t> opt_axis(int64_t a) {
  return a < 0 ? std::nullopt : std::optional<size_t>((size_t)a);
}

// Generic op dispatch by name.  ip = integer parameters, fp = float parameters.
//   reductions: ip[0] = axis or -1           log_softmax/argmax/argmin/concat/expand_dims: ip[0] = axis
//   squeeze: ip[0] = axis or -1              slice: ip = start0,end0,start1,end1,...
//   conv2d / conv2d_transpose: ip = sh,sw,ph,pw ; inputs = x,w[,bias]
//   max_pool2d: ip = kh,kw,sh,sw,ph,pw       view/broadcast_to: ip = shape
//   elu/mul_scalar/div_scalar/powf_scalar: fp[0] ; clip: fp[0],fp[1]
//   mse_loss/bce_with_logits: ip[0] = reduction (0 none,1 sum,2 mean) ; softmax_cross_entropy: ip = axis,reduction
template <class B>
Tensor<B> run_op(const std::string& name, const std::vector<Tensor<B>>& in, const std::vector<int64_t>& ip,
                 const std::vector<double>& fp) {
  auto need = [&](size_t n) {
    if (in.size() != n) throw Error::invalid_op(name + ": expected " + std::to_string(n) + " inputs");
  };
  auto ipa = [&](size_t i) -> int64_t {
    if (i >= ip.size()) throw Error::invalid_op(name + ": missing integer parameter");
    return ip[i];
  };
  auto fpa = [&](size_t i) -> float {
    if (i >= fp.size()) throw Error::invalid_op(name + ": missing float parameter");
    return (float)fp[i];
  };
  auto red = [&](int64_t r) { return r == 0 ? Reduction::None : (r == 1 ? Reduction::Sum : Reduction::Mean); };
#define RT_B2(n) if (name == #n) { need(2); return ops::n(in[0], in[1]); }
#define RT_U1(n) if (name == #n) { need(1); return ops::n(in[0]); }
#define RT_R1(n) if (name == #n) { need(1); return ops::n(in[0], opt_axis(ipa(0))); }
  RT_B2(matmul) RT_B2(mul) RT_B2(add) RT_B2(sub) RT_B2(div) RT_B2(powf) RT_B2(maximum) RT_B2(minimum)
  RT_U1(relu) RT_U1(sigmoid) RT_U1(abs) RT_U1(exp) RT_U1(ln) RT_U1(sqrt) RT_U1(tanh) RT_U1(softplus)
  RT_U1(square) RT_U1(sin) RT_U1(transpose)
  RT_R1(mean) RT_R1(sum) RT_R1(max) RT_R1(min) RT_R1(prod) RT_R1(logsumexp)
  RT_B2(equal) RT_B2(not_equal) RT_B2(greater) RT_B2(greater_equal) RT_B2(less) RT_B2(less_equal)
#undef RT_B2
#undef RT_U1
#undef RT_R1
  // cos / tan exist only at the Backend level in the reference (src/backend/mod.rs:486-507; its ops:: front-end has no
  // cos/tan): "backend_cos" calls B::cos, "backend_cos_backward" calls B::cos_backward with an Op holding x (inputs x, g).
  if (name == "backend_cos") { need(1); return Tensor<B>(B::cos(in[0].data()), false); }
  if (name == "backend_tan") { need(1); return Tensor<B>(B::tan(in[0].data()), false); }
  if (name == "backend_cos_backward" || name == "backend_tan_backward") {
    need(2);
    const bool is_cos = name == "backend_cos_backward";
    Op<B> op(OpType(is_cos ? OpType::Cos : OpType::Tan), {in[0]}, nullptr);
    return Tensor<B>(is_cos ? B::cos_backward(op, in[1].data()) : B::tan_backward(op, in[1].data()), false);
  }
  // random factories (no inputs): ip = shape (kaiming_uniform: fan_in, then the shape), fp = distribution parameters
  if (name == "manual_seed") { need(0); B::manual_seed((uint64_t)ipa(0)); return Tensor<B>(B::zeros(Shape{}), false); }
  if (name == "random_uniform") { need(0); return Tensor<B>(B::random_uniform(to_shape(ip.data(), (int)ip.size()), fpa(0), fpa(1)), false); }
  if (name == "random_normal") { need(0); return Tensor<B>(B::random_normal(to_shape(ip.data(), (int)ip.size()), fpa(0), fpa(1)), false); }
  if (name == "bernoulli") { need(0); return Tensor<B>(B::bernoulli(to_shape(ip.data(), (int)ip.size()), fpa(0)), false); }
  if (name == "kaiming_uniform") {
    need(0);
    return Tensor<B>::kaiming_uniform((size_t)ipa(0), to_shape(ip.data() + 1, (int)ip.size() - 1), fpa(0) != 0.f);
  }
  if (name == "elu") { need(1); return ops::elu(in[0], fpa(0)); }
  if (name == "mul_scalar") { need(1); return ops::mul_scalar(in[0], fpa(0)); }
  if (name == "div_scalar") { need(1); return ops::div_scalar(in[0], fpa(0)); }
  if (name == "powf_scalar") { need(1); return ops::powf_scalar(in[0], fpa(0)); }
  if (name == "clip") { need(1); return ops::clip(in[0], fpa(0), fpa(1)); }
  if (name == "log_softmax") { need(1); return ops::log_softmax(in[0], (size_t)ipa(0)); }
  if (name == "argmax") { need(1); return ops::argmax(in[0], (size_t)ipa(0)); }
  if (name == "argmin") { need(1); return ops::argmin(in[0], (size_t)ipa(0)); }
  if (name == "expand_dims") { need(1); return ops::expand_dims(in[0], (size_t)ipa(0)); }
  if (name == "squeeze") { need(1); return ops::squeeze(in[0], opt_axis(ipa(0))); }
  if (name == "concat") { return ops::concat<B>(in, (size_t)ipa(0)); }
  if (name == "view") { need(1); return ops::view(in[0], to_shape(ip.data(), (int)ip.size())); }
  if (name == "broadcast_to") { need(1); return ops::broadcast_to(in[0], to_shape(ip.data(), (int)ip.size())); }
  if (name == "slice") {
    need(1);
    std::vector<Range> r;
    for (size_t i = 0; i + 1 < ip.size(); i += 2) r.push_back({(size_t)ip[i], (size_t)ip[i + 1]});
    return ops::slice(in[0], r);
  }
  if (name == "conv2d" || name == "conv2d_transpose") {
    if (in.size() != 2 && in.size() != 3) throw Error::invalid_op(name + ": expected 2 or 3 inputs");
    Pair s{(size_t)ipa(0), (size_t)ipa(1)}, p{(size_t)ipa(2), (size_t)ipa(3)};
    const Tensor<B>* bias = in.size() == 3 ? &in[2] : nullptr;
    return name == "conv2d" ? ops::conv2d(in[0], in[1], bias, s, p) : ops::conv2d_transpose(in[0], in[1], bias, s, p);
  }
  if (name == "max_pool2d") {
    need(1);
    return ops::max_pool2d(in[0], {(size_t)ipa(0), (size_t)ipa(1)}, {(size_t)ipa(2), (size_t)ipa(3)},
                           {(size_t)ipa(4), (size_t)ipa(5)});
  }
  if (name == "mse_loss") { need(2); return ops::mse_loss(in[0], in[1], red(ipa(0))); }
  if (name == "binary_cross_entropy_with_logits") {
    need(2);
    return ops::binary_cross_entropy_with_logits(in[0], in[1], red(ipa(0)));
  }
  if (name == "softmax_cross_entropy") {
    need(2);
    return ops::softmax_cross_entropy(in[0], in[1], (size_t)ipa(0), red(ipa(1)));
  }
  throw Error::invalid_op("unknown op '" + name + "'");
}

template <class B, class F>
int guarded(F f) {
  auto& reg = Registry<B>::instance();
  try {
    f(reg);
    return 0;
  } catch (const Error& e) {
    reg.last_error = e.msg;
    return (int)e.kind;
  } catch (const std::exception& e) {
    reg.last_error = e.what();
    return (int)ErrorKind::InternalLogicError;
  }
}

}  // namespace capi
}  // namespace rt

#define RT_DEFINE_ENGINE_CAPI(P, BK)                                                                          \
  extern "C" {                                                                                                \
  const char* P##_last_error() { return rt::capi::Registry<BK>::instance().last_error.c_str(); }              \
  int P##_tensor_from_host(const float* data, const int64_t* shape, int ndim, int requires_grad,              \
                           int64_t* out) {                                                                    \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      rt::Shape s = rt::capi::to_shape(shape, ndim);                                                          \
      std::vector<float> v(data, data + rt::shape_numel(s));                                                  \
      *out = r.put(rt::Tensor<BK>::from_vec(std::move(v), s, requires_grad != 0));                            \
    });                                                                                                       \
  }                                                                                                           \
  int P##_tensor_free(int64_t h) {                                                                            \
    return rt::capi::guarded<BK>([&](auto& r) { r.tensors.erase(h); });                                       \
  }                                                                                                           \
  int P##_tensor_ndim(int64_t h, int* ndim) {                                                                 \
    return rt::capi::guarded<BK>([&](auto& r) { *ndim = (int)r.get(h).shape().size(); });                     \
  }                                                                                                           \
  int P##_tensor_shape(int64_t h, int64_t* shape) {                                                           \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      rt::Shape s = r.get(h).shape();                                                                         \
      for (size_t i = 0; i < s.size(); ++i) shape[i] = (int64_t)s[i];                                         \
    });                                                                                                       \
  }                                                                                                           \
  int P##_tensor_to_host(int64_t h, float* out, int64_t cap) {                                                \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      std::vector<float> v = r.get(h).to_vec();                                                               \
      if ((int64_t)v.size() > cap) throw rt::Error::invalid_op("tensor_to_host: buffer too small");           \
      if (!v.empty()) std::memcpy(out, v.data(), v.size() * sizeof(float));                                   \
    });                                                                                                       \
  }                                                                                                           \
  int P##_tensor_update_from_host(int64_t h, const float* data, int64_t n) {                                  \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      BK::update_from_host(r.get(h).data_mut(), std::vector<float>(data, data + n));                          \
    });                                                                                                       \
  }                                                                                                           \
  int P##_tensor_has_grad(int64_t h, int* has) {                                                              \
    return rt::capi::guarded<BK>([&](auto& r) { *has = r.get(h).grad() ? 1 : 0; });                           \
  }                                                                                                           \
  int P##_tensor_grad(int64_t h, int64_t* out) {                                                              \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& t = r.get(h);                                                                                     \
      if (!t.grad()) throw rt::Error(rt::ErrorKind::NoGradientError, "tensor has no gradient");               \
      *out = r.put(rt::Tensor<BK>(*t.grad(), false));                                                         \
    });                                                                                                       \
  }                                                                                                           \
  int P##_tensor_set_grad(int64_t h, int64_t grad_h) {                                                        \
    return rt::capi::guarded<BK>([&](auto& r) { r.get(h).set_grad(r.get(grad_h).data()); });                  \
  }                                                                                                           \
  int P##_tensor_zero_grad(int64_t h) {                                                                       \
    return rt::capi::guarded<BK>([&](auto& r) { r.get(h).zero_grad(); });                                     \
  }                                                                                                           \
  int P##_tensor_requires_grad(int64_t h, int* rg) {                                                          \
    return rt::capi::guarded<BK>([&](auto& r) { *rg = r.get(h).requires_grad() ? 1 : 0; });                   \
  }                                                                                                           \
  int P##_op(const char* name, const int64_t* inputs, int n_in, const int64_t* ip, int n_ip,                  \
             const double* fp, int n_fp, int64_t* out) {                                                      \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      std::vector<rt::Tensor<BK>> in;                                                                         \
      for (int i = 0; i < n_in; ++i) in.push_back(r.get(inputs[i]));                                          \
      std::vector<int64_t> ipv(ip, ip + n_ip);                                                                \
      std::vector<double> fpv(fp, fp + n_fp);                                                                 \
      *out = r.put(rt::capi::run_op<BK>(name, in, ipv, fpv));                                                 \
    });                                                                                                       \
  }                                                                                                           \
  /* data::get_batch / get_random_batch (src/data.rs:125-209): n_idx > 0 -> the given rows; else `batch` random rows */  \
  int P##_get_batch(int64_t xh, int64_t yh, const int64_t* idx, int n_idx, int64_t batch, uint64_t seed,      \
                    int64_t* out_x, int64_t* out_y) {                                                         \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto res = n_idx > 0 ? rt::data::get_batch(r.get(xh), r.get(yh), std::vector<size_t>(idx, idx + n_idx)) \
                           : rt::data::get_random_batch(r.get(xh), r.get(yh), (size_t)batch, seed);           \
      *out_x = r.put(res.first);                                                                              \
      *out_y = r.put(res.second);                                                                             \
    });                                                                                                       \
  }                                                                                                           \
  int P##_backward(int64_t h) {                                                                               \
    return rt::capi::guarded<BK>([&](auto& r) { r.get(h).backward(); });                                      \
  }                                                                                                           \
  /* Calls the backward closure of the op that produced `h` with an explicit upstream                         \
     gradient (any shape), returning one tensor per op input. */                                              \
  int P##_op_backward(int64_t h, int64_t grad_h, int64_t* outs, int cap, int* n_out) {                        \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& t = r.get(h);                                                                                     \
      if (!t.inner->op) throw rt::Error::invalid_op("op_backward: tensor has no op");                         \
      auto grads = t.inner->op->backward_fn(*t.inner->op, r.get(grad_h).data());                              \
      if ((int)grads.size() > cap) throw rt::Error::invalid_op("op_backward: output array too small");        \
      *n_out = (int)grads.size();                                                                             \
      for (size_t i = 0; i < grads.size(); ++i) outs[i] = r.put(rt::Tensor<BK>(std::move(grads[i]), false));  \
    });                                                                                                       \
  }                                                                                                           \
  /* optimizers: kind 0 Sgd(lr) 1 Adam(lr,b1,b2,eps) 2 MomentumSGD(lr,mu) 3 AdaGrad(lr,eps) */                \
  int P##_optim_create(int kind, const int64_t* params, int n, const double* hp, int n_hp, int64_t* out) {    \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      std::vector<rt::Tensor<BK>> ps;                                                                         \
      for (int i = 0; i < n; ++i) ps.push_back(r.get(params[i]));                                             \
      auto hpa = [&](int i) {                                                                                 \
        if (i >= n_hp) throw rt::Error::invalid_op("optim_create: missing hyper-parameter");                  \
        return (float)hp[i];                                                                                  \
      };                                                                                                      \
      typename rt::capi::Registry<BK>::Optim o;                                                               \
      o.kind = kind;                                                                                          \
      if (kind == 0) o.sgd = std::make_shared<rt::optim::Sgd<BK>>(ps, hpa(0));                                \
      else if (kind == 1) o.adam = std::make_shared<rt::optim::Adam<BK>>(ps, hpa(0), hpa(1), hpa(2), hpa(3)); \
      else if (kind == 2) o.mom = std::make_shared<rt::optim::MomentumSGD<BK>>(ps, hpa(0), hpa(1));           \
      else if (kind == 3) o.ada = std::make_shared<rt::optim::AdaGrad<BK>>(ps, hpa(0), hpa(1));               \
      else throw rt::Error::invalid_op("optim_create: unknown kind");                                         \
      r.optims[r.next] = o;                                                                                   \
      *out = r.next++;                                                                                        \
    });                                                                                                       \
  }                                                                                                           \
  int P##_optim_step(int64_t h) {                                                                             \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& o = r.optims.at(h);                                                                               \
      if (o.sgd) o.sgd->step();                                                                               \
      if (o.adam) o.adam->step();                                                                             \
      if (o.mom) o.mom->step();                                                                               \
      if (o.ada) o.ada->step();                                                                               \
    });                                                                                                       \
  }                                                                                                           \
  int P##_optim_zero_grad(int64_t h) {                                                                        \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& o = r.optims.at(h);                                                                               \
      if (o.sgd) o.sgd->zero_grad();                                                                          \
      if (o.adam) o.adam->zero_grad();                                                                        \
      if (o.mom) rt::optim::zero_grad_all(o.mom->parameters);                                                 \
      if (o.ada) o.ada->zero_grad();                                                                          \
    });                                                                                                       \
  }                                                                                                           \
  /* which: 0 = first state (m / velocity / accumulator), 1 = second state (v) */                             \
  int P##_optim_state(int64_t h, int which, int idx, int64_t* out) {                                          \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& o = r.optims.at(h);                                                                               \
      if (o.adam) *out = r.put(rt::Tensor<BK>(which == 0 ? o.adam->m_states.at(idx) : o.adam->v_states.at(idx), false)); \
      else if (o.mom) *out = r.put(rt::Tensor<BK>(o.mom->velocities.at(idx), false));                         \
      else if (o.ada) *out = r.put(rt::Tensor<BK>(o.ada->accumulated_sq_grad.at(idx), false));                \
      else throw rt::Error::invalid_op("optim_state: optimizer has no state");                                \
    });                                                                                                       \
  }                                                                                                           \
  int P##_optim_free(int64_t h) {                                                                             \
    return rt::capi::guarded<BK>([&](auto& r) { r.optims.erase(h); });                                        \
  }                                                                                                           \
  /* workloads */                                                                                             \
  int P##_trainer_create(int config, const int64_t* dims, int nd, int64_t* out) {                             \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      std::vector<size_t> d(dims, dims + nd);                                                                 \
      r.trainers[r.next] = std::make_shared<rt::models::Trainer<BK>>(rt::models::make_workload<BK>(config, d)); \
      *out = r.next++;                                                                                        \
    });                                                                                                       \
  }                                                                                                           \
  int P##_trainer_free(int64_t h) {                                                                           \
    return rt::capi::guarded<BK>([&](auto& r) { r.trainers.erase(h); });                                      \
  }                                                                                                           \
  int P##_trainer_num_params(int64_t h, int* n) {                                                             \
    return rt::capi::guarded<BK>([&](auto& r) { *n = (int)r.trainers.at(h)->w.params.size(); });              \
  }                                                                                                           \
  int P##_trainer_param(int64_t h, int i, int64_t* out) {                                                     \
    return rt::capi::guarded<BK>([&](auto& r) { *out = r.put(r.trainers.at(h)->w.params.at(i)); });           \
  }                                                                                                           \
  int P##_trainer_set_hyper(int64_t h, const double* hp, int n) {                                             \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& w = r.trainers.at(h)->w;                                                                          \
      if (n > 0) w.lr = (float)hp[0];                                                                         \
      if (n > 1) w.beta1 = (float)hp[1];                                                                      \
      if (n > 2) w.beta2 = (float)hp[2];                                                                      \
      if (n > 3) w.eps = (float)hp[3];                                                                        \
      if (n > 4) w.momentum = (float)hp[4];                                                                   \
    });                                                                                                       \
  }                                                                                                           \
  /* mode: 0 = forward only, 1 = forward+backward(+clip), 2 = full step */                                    \
  int P##_trainer_run(int64_t h, const int64_t* inputs, int n_in, int mode, int64_t* loss_out) {              \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& tr = *r.trainers.at(h);                                                                           \
      std::vector<rt::Tensor<BK>> in;                                                                         \
      for (int i = 0; i < n_in; ++i) in.push_back(r.get(inputs[i]));                                          \
      rt::Tensor<BK> loss = mode == 0 ? rt::models::forward_loss(tr.w, in)                                    \
                                      : (mode == 1 ? tr.forward_backward(in) : tr.step(in));                  \
      *loss_out = r.put(loss);                                                                                \
    });                                                                                                       \
  }                                                                                                           \
  int P##_trainer_optimizer_step(int64_t h) {                                                                 \
    return rt::capi::guarded<BK>([&](auto& r) { r.trainers.at(h)->optimizer_step(); });                       \
  }                                                                                                           \
  int P##_trainer_optim_state(int64_t h, int which, int idx, int64_t* out) {                                  \
    return rt::capi::guarded<BK>([&](auto& r) {                                                               \
      auto& tr = *r.trainers.at(h);                                                                           \
      tr.ensure_optimizer();                                                                                  \
      if (tr.adam) *out = r.put(rt::Tensor<BK>(which == 0 ? tr.adam->m_states.at(idx) : tr.adam->v_states.at(idx), false)); \
      else if (tr.msgd) *out = r.put(rt::Tensor<BK>(tr.msgd->velocities.at(idx), false));                     \
      else throw rt::Error::invalid_op("trainer has no optimizer state");                                     \
    });                                                                                                       \
  }                                                                                                           \
  }
