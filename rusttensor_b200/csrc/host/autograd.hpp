// Define-by-run reverse-mode autograd, generic over a Backend type.
//
// This header restates, in C++, the host-side layer that sits above the
// `Backend` trait of the reference library:
//   * Tensor / TensorData            -> src/tensor.rs:60-68, 731-744
//   * Tensor::backward / topo sort   -> src/tensor.rs:1150-1260
//   * Tensor::add_grad / set_grad    -> src/tensor.rs:1026-1138
//   * OpType / Op                    -> src/graph.rs:9-64, 147-170
//   * op front-end (ops::*)          -> src/ops/mod.rs (one function per public op)
//   * generic new_with_op dispatch   -> src/tensor.rs:747-902
//   * Error / Reduction              -> src/error.rs:8-116
//
// A Backend `B` supplies `B::Storage` (value semantics: a copy behaves like a
// deep copy) and static functions with the same names and argument meaning as
// the reference trait (src/backend/mod.rs:14-656).  The engine never touches
// tensor bytes itself.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cmath>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <tuple>
#include <unordered_set>
#include <utility>
#include <type_traits>
#include <vector>

namespace rt {

using Shape = std::vector<size_t>;
using Pair = std::pair<size_t, size_t>;

inline size_t shape_numel(const Shape& s) {
  size_t n = 1;
  for (size_t d : s) n *= d;
  return n;
}
inline std::string shape_str(const Shape& s) {
  std::string r = "[";
  for (size_t i = 0; i < s.size(); ++i) r += (i ? ", " : "") + std::to_string(s[i]);
  return r + "]";
}

// ---- src/error.rs:8-98 ------------------------------------------------------
enum class ErrorKind : int {
  ShapeMismatch = 1,
  IncompatibleShapes = 2,
  InvalidIndex = 3,
  InvalidOperation = 4,
  InternalLogicError = 5,
  DimensionMismatch = 6,
  CudaError = 7,
  OutOfMemory = 8,
  Unimplemented = 9,
  EmptyTensor = 10,
  ShapeError = 11,
  NoGradientError = 12,
  GradientCheckError = 13,
  Timeout = 14,
  Nccl = 15,
  InitializationError = 16,
};

struct Error : public std::exception {
  ErrorKind kind;
  std::string msg;
  Error(ErrorKind k, std::string m) : kind(k), msg(std::move(m)) {}
  const char* what() const noexcept override { return msg.c_str(); }
  static Error shape_mismatch(const Shape& expected, const Shape& actual) {
    return Error(ErrorKind::ShapeMismatch,
                 "Shape mismatch: expected " + shape_str(expected) + ", got " + shape_str(actual));
  }
  static Error incompatible(const std::string& op, const Shape& a, const Shape& b) {
    return Error(ErrorKind::IncompatibleShapes,
                 "Incompatible shapes for " + op + ": " + shape_str(a) + " and " + shape_str(b));
  }
  static Error invalid_index(size_t ax) {
    return Error(ErrorKind::InvalidIndex, "Invalid index [" + std::to_string(ax) + "]");
  }
  static Error invalid_op(const std::string& m) { return Error(ErrorKind::InvalidOperation, m); }
  static Error internal(const std::string& m) { return Error(ErrorKind::InternalLogicError, m); }
  static Error unimplemented(const std::string& m) { return Error(ErrorKind::Unimplemented, m); }
};

// src/error.rs:109-116
enum class Reduction { None, Sum, Mean };

struct Range {
  size_t start, end;
};

// ---- src/graph.rs:9-64 ------------------------------------------------------
struct OpType {
  enum Kind {
    Matmul, Mul, Add, Mean, Relu, LogSoftmax, Sum, Sub, Div, Exp, Ln, Broadcast, View, Abs,
    Sigmoid, Sqrt, Tanh, Softplus, Max, Min, Prod, LogSumExp, ArgMax, ArgMin, Powf, Square,
    Maximum, Minimum, Elu, Transpose, Sin, Cos, Tan, Conv2d, MaxPool2D, Conv2DTranspose, Slice,
    Concat, ExpandDims, Squeeze, Clip, DivScalar, MulScalar,
    FusedReluMaxPool2D, FusedSoftmaxNll, FusedLstmCellC, FusedLstmCellH, FusedConvReluMaxPool2D  // fused forward ops added beside the reference's (ops::fused_*)
  } kind;
  std::optional<size_t> axis;          // Mean/Sum/Max/Min/Prod/LogSumExp(Option), LogSoftmax/ArgMax/...
  float scalar = 0.f;                  // Elu(alpha), MulScalar, DivScalar
  float min_val = 0.f, max_val = 0.f;  // Clip
  Pair stride{1, 1}, padding{0, 0}, kernel_size{1, 1};
  Shape input_shape;                   // Slice, Squeeze(original_input_shape)
  std::vector<Range> ranges;           // Slice
  std::vector<Shape> input_shapes;     // Concat
  OpType(Kind k) : kind(k) {}
  static OpType with_axis(Kind k, std::optional<size_t> ax) {
    OpType t(k);
    t.axis = ax;
    return t;
  }
  const char* name() const {
    static const char* n[] = {"Matmul", "Mul", "Add", "Mean", "Relu", "LogSoftmax", "Sum", "Sub",
      "Div", "Exp", "Ln", "Broadcast", "View", "Abs", "Sigmoid", "Sqrt", "Tanh", "Softplus", "Max",
      "Min", "Prod", "LogSumExp", "ArgMax", "ArgMin", "Powf", "Square", "Maximum", "Minimum", "Elu",
      "Transpose", "Sin", "Cos", "Tan", "Conv2d", "MaxPool2D", "Conv2DTranspose", "Slice", "Concat",
      "ExpandDims", "Squeeze", "Clip", "DivScalar", "MulScalar", "FusedReluMaxPool2D", "FusedSoftmaxNll", "FusedLstmCellC", "FusedLstmCellH", "FusedConvReluMaxPool2D"};
    return n[(int)kind];
  }
};

template <class B> class Tensor;

// ---- src/graph.rs:147-170 ---------------------------------------------------
template <class B>
struct Op {
  using Storage = typename B::Storage;
  using BackwardFn = std::function<std::vector<Storage>(const Op<B>&, const Storage&)>;
  OpType op_type;
  std::vector<Tensor<B>> inputs;
  BackwardFn backward_fn;
  std::optional<Storage> cached_outputs;
  Op(OpType t, std::vector<Tensor<B>> in, BackwardFn fn)
      : op_type(std::move(t)), inputs(std::move(in)), backward_fn(std::move(fn)) {}
};

inline size_t next_tensor_id() {
  static size_t counter = 0;
  return counter++;
}

// ---- src/tensor.rs:60-68 ----------------------------------------------------
template <class B>
struct TensorData {
  size_t id;
  typename B::Storage data;
  std::optional<typename B::Storage> grad;
  bool requires_grad;
  std::shared_ptr<Op<B>> op;
};

// A backend may add a product's weight gradient to the gradient the weight already holds (a weight used at every timestep
// of a recurrent layer) inside the product itself, instead of returning it for a separate addition.
template <class B, class = void>
struct HasAccumulatingMatmul : std::false_type {};
template <class B>
struct HasAccumulatingMatmul<B, std::void_t<decltype(&B::matmul_backward_accumulate)>> : std::true_type {};

template <class B>
class Tensor {
 public:
  using Storage = typename B::Storage;
  std::shared_ptr<TensorData<B>> inner;

  Tensor() = default;
  // src/tensor.rs:731-744
  Tensor(Storage data, bool requires_grad)
      : inner(std::make_shared<TensorData<B>>(
            TensorData<B>{next_tensor_id(), std::move(data), std::nullopt, requires_grad, nullptr})) {}

  static Tensor zeros(const Shape& s, bool rg) { return Tensor(B::zeros(s), rg); }
  // src/tensor.rs:953-960
  static Tensor kaiming_uniform(size_t fan_in, const Shape& s, bool rg) { return Tensor(B::kaiming_uniform(fan_in, s), rg); }
  static Tensor ones(const Shape& s, bool rg) { return Tensor(B::ones(s), rg); }
  static Tensor from_vec(std::vector<float> v, const Shape& s, bool rg) {
    return Tensor(B::from_vec(std::move(v), s), rg);
  }

  const Storage& data() const { return inner->data; }
  Storage& data_mut() const { return inner->data; }
  Shape shape() const { return B::shape(inner->data); }
  size_t size() const { return B::size(inner->data); }
  bool requires_grad() const { return inner->requires_grad; }
  size_t id() const { return inner->id; }
  const std::optional<Storage>& grad() const { return inner->grad; }
  Storage& grad_mut() const { return *inner->grad; }  // only valid while grad() holds a value
  std::vector<float> to_vec() const { return B::copy_to_host(inner->data); }
  std::vector<float> grad_vec() const {
    if (!inner->grad) throw Error(ErrorKind::NoGradientError, "tensor has no gradient");
    return B::copy_to_host(*inner->grad);
  }
  void set_op(Op<B> op) const { inner->op = std::make_shared<Op<B>>(std::move(op)); }

  // src/tensor.rs:1026-1040 (the reference panics on a shape mismatch)
  void set_grad(std::optional<Storage> g) const {
    if (g && B::shape(inner->data) != B::shape(*g))
      throw Error::shape_mismatch(B::shape(inner->data), B::shape(*g));
    inner->grad = std::move(g);
  }
  // src/tensor.rs:1043-1046
  void zero_grad() const { inner->grad.reset(); }

  // src/tensor.rs:1049-1138: first contribution is stored, later ones are
  // accumulated with one B::add into a fresh storage.
  void add_grad(Storage g) const {
    Shape ds = B::shape(inner->data), gs = B::shape(g);
    if (ds != gs) throw Error::incompatible("add_grad on Tensor ID " + std::to_string(id()), ds, gs);
    if (inner->grad) {
      Storage existing = *inner->grad;
      inner->grad = B::add(existing, g);
    } else {
      inner->grad = std::move(g);
    }
  }

  // src/tensor.rs:1225-1260: DFS post-order over op.inputs (leaves first, root
  // last).  Iterative so that deep unrolled graphs do not exhaust the stack;
  // the visiting order is the recursive one.
  std::vector<Tensor<B>> build_topo_sort() const {
    std::vector<Tensor<B>> sorted;
    std::unordered_set<size_t> visited, visiting;
    struct Frame { Tensor<B> node; size_t next; };
    std::vector<Frame> stack;
    auto enter = [&](const Tensor<B>& n) {
      if (visited.count(n.id())) return;
      if (!visiting.insert(n.id()).second)
        throw Error::internal("Cycle detected in computation graph involving Tensor ID " +
                              std::to_string(n.id()));
      stack.push_back({n, 0});
    };
    enter(*this);
    while (!stack.empty()) {
      Frame& f = stack.back();
      const auto& op = f.node.inner->op;
      if (op && f.next < op->inputs.size()) {
        Tensor<B> child = op->inputs[f.next++];
        enter(child);
      } else {
        visiting.erase(f.node.id());
        visited.insert(f.node.id());
        sorted.push_back(f.node);
        stack.pop_back();
      }
    }
    return sorted;
  }

  // src/tensor.rs:1150-1220
  // Optional observer (not in the reference): called by backward() when the walk reaches a leaf that requires a
  // gradient, i.e. when that gradient is final.  The data-parallel trainer uses it to start exchanging the gradients
  // that are ready while the rest of the backward pass is still being enqueued.
  static std::function<void(const Tensor&)>& leaf_ready_hook() {
    static thread_local std::function<void(const Tensor&)> hook;
    return hook;
  }

  void backward() const {
    if (!requires_grad()) return;
    if (size() == 1) {
      if (!inner->grad) set_grad(B::ones(Shape{}));
    } else if (!inner->grad) {
      throw Error::invalid_op(
          "backward() called on non-scalar tensor without pre-existing gradient. Seed gradient required.");
    }
    auto nodes = build_topo_sort();
    std::unordered_set<size_t> visited;
    for (auto it = nodes.rbegin(); it != nodes.rend(); ++it) {
      const Tensor<B>& node = *it;
      if (!visited.insert(node.id()).second) continue;
      std::shared_ptr<Op<B>> op = node.inner->op;
      if (!op) {
        // every consumer of this leaf has been processed: its gradient is final
        if (node.inner->grad && node.requires_grad() && leaf_ready_hook()) leaf_ready_hook()(node);
        continue;
      }
      if (!node.inner->grad) continue;
      Storage out_grad = *node.inner->grad;  // value copy, as the reference clones
      std::vector<Storage> grads = op->backward_fn(*op, out_grad);
      if (grads.size() != op->inputs.size())
        throw Error::invalid_op(std::string("Backward function for op ") + op->op_type.name() +
                                " returned " + std::to_string(grads.size()) + " gradients, expected " +
                                std::to_string(op->inputs.size()));
      for (size_t i = 0; i < grads.size(); ++i) {
        if (!op->inputs[i].requires_grad()) continue;
        if constexpr (HasAccumulatingMatmul<B>::value) {
          if (B::is_accumulated(grads[i])) continue;  // the closure has added its gradient to the existing one itself
        }
        op->inputs[i].add_grad(std::move(grads[i]));
      }
    }
  }

  // Drops the graph reachable from this tensor (used between steps so that
  // device buffers return to the pool).
  void detach_graph() const { inner->op.reset(); }

  // src/tensor.rs:747-902: generic dispatch on the op type.
  static Tensor new_with_op(Storage data, bool requires_grad, std::optional<OpType> op_type,
                            std::vector<Tensor<B>> inputs) {
    Tensor t(std::move(data), requires_grad);
    if (op_type) {
      t.set_op(Op<B>(*op_type, std::move(inputs), [](const Op<B>& op, const Storage& g) {
        return dispatch_backward(op, g);
      }));
    }
    return t;
  }

  static std::vector<Storage> dispatch_backward(const Op<B>& op, const Storage& g) {
    auto two = [](std::pair<Storage, Storage> p) {
      return std::vector<Storage>{std::move(p.first), std::move(p.second)};
    };
    auto one = [](Storage s) { return std::vector<Storage>{std::move(s)}; };
    switch (op.op_type.kind) {
      case OpType::Add: return two(B::add_backward(op, g));
      case OpType::Mul: return two(B::mul_backward(op, g));
      case OpType::Matmul: return two(B::matmul_backward(op, g));
      case OpType::Mean: return one(B::mean_backward(op, g));
      case OpType::Relu: return one(B::relu_backward(op, g));
      case OpType::LogSoftmax: return one(B::log_softmax_backward(op, g));
      case OpType::Sum: return one(B::sum_backward(op, g));
      case OpType::Max: return one(B::max_backward(op, g));
      case OpType::Min: return one(B::min_backward(op, g));
      case OpType::Prod: return one(B::prod_backward(op, g));
      case OpType::LogSumExp: return one(B::logsumexp_backward(op, g));
      case OpType::ArgMax: throw Error::unimplemented("Backward pass for ArgMax is not implemented");
      case OpType::ArgMin: throw Error::unimplemented("Backward pass for ArgMin is not implemented");
      case OpType::Sub: return two(B::sub_backward(op, g));
      case OpType::Div: return two(B::div_backward(op, g));
      case OpType::Exp: return one(B::exp_backward(op, g));
      case OpType::Ln: return one(B::ln_backward(op, g));
      case OpType::Broadcast:  // src/tensor.rs:785-794
        return one(B::unbroadcast(g, B::shape(op.inputs[0].data())));
      case OpType::View: {  // src/tensor.rs:795-802
        Storage grad = g;
        B::set_shape(grad, B::shape(op.inputs[0].data()));
        return one(std::move(grad));
      }
      case OpType::Abs: return one(B::abs_backward(op, g));
      case OpType::Sigmoid: return one(B::sigmoid_backward(op, g));
      case OpType::Tanh: return one(B::tanh_backward(op, g));
      case OpType::Sqrt: return one(B::sqrt_backward(op, g));
      case OpType::Softplus: return one(B::softplus_backward(op, g));
      case OpType::Powf: return two(B::powf_backward(op, g));
      case OpType::Square: return one(B::square_backward(op, g));
      case OpType::Maximum: return two(B::maximum_backward(op, g));
      case OpType::Minimum: return two(B::minimum_backward(op, g));
      case OpType::Elu: return one(B::elu_backward(op, g));
      case OpType::Transpose: return one(B::transpose(g));
      case OpType::Sin: return one(B::sin_backward(op, g));
      case OpType::Cos: throw Error::unimplemented("Backward pass for Cos is not yet implemented");
      case OpType::Tan: throw Error::unimplemented("Backward pass for Tan is not yet implemented");
      case OpType::Concat: return B::concat_backward(op, g);
      case OpType::Slice: return one(B::slice_backward(op, g));
      case OpType::ExpandDims: return one(B::expand_dims_backward(op, g));
      case OpType::Squeeze: return one(B::squeeze_backward(op, g));
      case OpType::Clip: return one(B::clip_backward(op, g));
      case OpType::MulScalar: return one(B::mul_scalar(g, op.op_type.scalar));
      case OpType::DivScalar:
        throw Error::invalid_op("Backward pass for DivScalar operation not implemented yet");
      case OpType::Conv2DTranspose:
        throw Error::unimplemented("Backward pass for Conv2DTranspose is not yet implemented");
      default:
        throw Error::internal(std::string("new_with_op: unsupported op type ") + op.op_type.name());
    }
  }

  // Tensor methods used by the examples (src/tensor.rs view/broadcast_to wrappers).
  Tensor view(const Shape& s) const;
  Tensor broadcast_to(const Shape& s) const;
};

// =============================================================================
// ops:: front-end (src/ops/mod.rs).  Each function calls the backend forward,
// creates the output tensor and, when a gradient is required, attaches an Op
// whose closure calls the backend backward.
// =============================================================================
namespace ops {

template <class B> using St = typename B::Storage;
template <class B> using Grads = std::vector<typename B::Storage>;

// src/ops/mod.rs:127-182.  The closure calls transpose twice and matmul twice.
template <class B>
Tensor<B> matmul(const Tensor<B>& a, const Tensor<B>& b) {
  Shape as = a.shape(), bs = b.shape();
  if (as.size() != 2 || bs.size() != 2)
    throw Error(ErrorKind::DimensionMismatch,
                "Dimension mismatch: expected 2, got " + std::to_string(std::max(as.size(), bs.size())));
  if (as[1] != bs[0]) throw Error::incompatible("matmul", as, bs);
  St<B> out = B::matmul(a.data(), b.data());
  bool rg = a.requires_grad() || b.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    t.set_op(Op<B>(OpType(OpType::Matmul), {a, b}, [](const Op<B>& op, const St<B>& g) {
      if constexpr (HasAccumulatingMatmul<B>::value) {
        const Tensor<B>& wb = op.inputs[1];
        if (wb.requires_grad() && wb.grad() && B::accumulates_well(wb.data())) {
          St<B> da = B::matmul_backward_accumulate(op, g, wb.grad_mut());
          return Grads<B>{std::move(da), B::unused_grad(B::shape(wb.data()))};
        }
      }
      auto p = B::matmul_closure_backward(op, g);
      return Grads<B>{std::move(p.first), std::move(p.second)};
    }));
  }
  return t;
}

// src/ops/mod.rs:190-261
template <class B>
Tensor<B> conv2d(const Tensor<B>& input, const Tensor<B>& weights, const Tensor<B>* bias, Pair stride,
                 Pair padding) {
  St<B> out = B::conv2d(input.data(), weights.data(), bias ? &bias->data() : nullptr, stride, padding);
  bool rg = input.requires_grad() || weights.requires_grad() || (bias && bias->requires_grad());
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Conv2d);
    ot.stride = stride;
    ot.padding = padding;
    Tensor<B> b = bias ? *bias : Tensor<B>(B::zeros(Shape{weights.shape()[0]}), false);
    t.set_op(Op<B>(ot, {input, weights, b}, [](const Op<B>& op, const St<B>& g) {
      auto r = B::conv2d_backward(op.inputs[0].data(), op.inputs[1].data(), g, op.op_type.stride,
                                  op.op_type.padding, op.inputs[0].requires_grad(),
                                  op.inputs[1].requires_grad(), op.inputs[2].requires_grad());
      St<B> gb = std::get<2>(r) ? std::move(*std::get<2>(r)) : B::zeros(Shape{0});
      return Grads<B>{std::move(std::get<0>(r)), std::move(std::get<1>(r)), std::move(gb)};
    }));
  }
  return t;
}

// src/ops/mod.rs:276-322
template <class B>
Tensor<B> conv2d_transpose(const Tensor<B>& input, const Tensor<B>& weights, const Tensor<B>* bias,
                           Pair stride, Pair padding) {
  St<B> out =
      B::conv2d_transpose(input.data(), weights.data(), bias ? &bias->data() : nullptr, stride, padding);
  bool rg = input.requires_grad() || weights.requires_grad() || (bias && bias->requires_grad());
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Conv2DTranspose);
    ot.stride = stride;
    ot.padding = padding;
    Tensor<B> b = bias ? *bias : Tensor<B>(B::zeros(Shape{weights.shape()[1]}), false);
    t.set_op(Op<B>(ot, {input, weights, b}, [](const Op<B>& op, const St<B>& g) {
      auto r = B::conv2d_transpose_backward(op.inputs[0].data(), op.inputs[1].data(), g,
                                            op.op_type.stride, op.op_type.padding,
                                            op.inputs[0].requires_grad(), op.inputs[1].requires_grad(),
                                            op.inputs[2].requires_grad());
      St<B> gb = std::get<2>(r) ? std::move(*std::get<2>(r)) : B::zeros(Shape{0});
      return Grads<B>{std::move(std::get<0>(r)), std::move(std::get<1>(r)), std::move(gb)};
    }));
  }
  return t;
}

// src/ops/mod.rs:337-372.  The index tensor is the Op's second input; its
// gradient slot is a zero tensor in the reference and is never accumulated
// (the index tensor does not require grad).
template <class B>
Tensor<B> max_pool2d(const Tensor<B>& input, Pair kernel, Pair stride, Pair padding) {
  auto r = B::max_pool2d(input.data(), kernel, stride, padding);
  bool rg = input.requires_grad();
  Tensor<B> t(std::move(r.first), rg);
  if (rg) {
    Tensor<B> idx(std::move(r.second), false);
    OpType ot(OpType::MaxPool2D);
    ot.kernel_size = kernel;
    ot.stride = stride;
    ot.padding = padding;
    t.set_op(Op<B>(ot, {input, idx}, [](const Op<B>& op, const St<B>& g) {
      St<B> gi = B::max_pool2d_backward(op, g);
      return Grads<B>{std::move(gi), B::unused_grad(B::shape(op.inputs[1].data()))};
    }));
  }
  return t;
}

#define RT_BINARY_OP(fname, fwd, bwd, KIND)                                                  \
  template <class B>                                                                         \
  Tensor<B> fname(const Tensor<B>& a, const Tensor<B>& b) {                                  \
    St<B> out = B::fwd(a.data(), b.data());                                                  \
    bool rg = a.requires_grad() || b.requires_grad();                                        \
    Tensor<B> t(std::move(out), rg);                                                         \
    if (rg) {                                                                                \
      t.set_op(Op<B>(OpType(OpType::KIND), {a, b}, [](const Op<B>& op, const St<B>& g) {     \
        auto p = B::bwd(op, g);                                                              \
        return Grads<B>{std::move(p.first), std::move(p.second)};                            \
      }));                                                                                   \
    }                                                                                        \
    return t;                                                                                \
  }
RT_BINARY_OP(mul, mul, mul_backward, Mul)                // src/ops/mod.rs:412-432
RT_BINARY_OP(add, add, add_backward, Add)                // src/ops/mod.rs:435-453
RT_BINARY_OP(sub, sub, sub_backward, Sub)                // src/ops/mod.rs:675-693
RT_BINARY_OP(div, div, div_backward, Div)                // src/ops/mod.rs:696-714
RT_BINARY_OP(powf, powf, powf_backward, Powf)            // src/ops/mod.rs:1125-1144
RT_BINARY_OP(maximum, maximum, maximum_backward, Maximum)  // src/ops/mod.rs:1201-1229
RT_BINARY_OP(minimum, minimum, minimum_backward, Minimum)  // src/ops/mod.rs:1240-1268
#undef RT_BINARY_OP

#define RT_UNARY_OP(fname, fwd, bwd, KIND)                                                   \
  template <class B>                                                                         \
  Tensor<B> fname(const Tensor<B>& x) {                                                      \
    St<B> out = B::fwd(x.data());                                                            \
    bool rg = x.requires_grad();                                                             \
    Tensor<B> t(std::move(out), rg);                                                         \
    if (rg) {                                                                                \
      t.set_op(Op<B>(OpType(OpType::KIND), {x}, [](const Op<B>& op, const St<B>& g) {        \
        return Grads<B>{B::bwd(op, g)};                                                      \
      }));                                                                                   \
    }                                                                                        \
    return t;                                                                                \
  }
RT_UNARY_OP(relu, relu, relu_backward, Relu)                  // src/ops/mod.rs:456-469
RT_UNARY_OP(sigmoid, sigmoid, sigmoid_backward, Sigmoid)      // src/ops/mod.rs:504-518
RT_UNARY_OP(abs, abs, abs_backward, Abs)                      // src/ops/mod.rs:598-611
RT_UNARY_OP(exp, exp, exp_backward, Exp)                      // src/ops/mod.rs:717-735
RT_UNARY_OP(ln, ln, ln_backward, Ln)                          // src/ops/mod.rs:738-756
RT_UNARY_OP(sqrt, sqrt, sqrt_backward, Sqrt)                  // src/ops/mod.rs:759-777
RT_UNARY_OP(tanh, tanh, tanh_backward, Tanh)                  // src/ops/mod.rs:999-1012
RT_UNARY_OP(softplus, softplus, softplus_backward, Softplus)  // src/ops/mod.rs:1015-1037
RT_UNARY_OP(square, square, square_backward, Square)          // src/ops/mod.rs:1161-1190
RT_UNARY_OP(sin, sin, sin_backward, Sin)                      // src/ops/mod.rs:1733-1745
#undef RT_UNARY_OP

// src/ops/mod.rs:483-501
template <class B>
Tensor<B> elu(const Tensor<B>& x, float alpha) {
  St<B> out = B::elu(x.data(), alpha);
  bool rg = x.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Elu);
    ot.scalar = alpha;
    t.set_op(Op<B>(ot, {x}, [](const Op<B>& op, const St<B>& g) { return Grads<B>{B::elu_backward(op, g)}; }));
  }
  return t;
}

// src/ops/mod.rs:521-545 (the forward output is cached on the Op)
template <class B>
Tensor<B> log_softmax(const Tensor<B>& x, size_t axis) {
  St<B> out = B::log_softmax(x.data(), axis);
  bool rg = x.requires_grad();
  Tensor<B> t(out, rg);
  if (rg) {
    Op<B> op(OpType::with_axis(OpType::LogSoftmax, axis), {x},
             [](const Op<B>& o, const St<B>& g) { return Grads<B>{B::log_softmax_backward(o, g)}; });
    op.cached_outputs = std::move(out);
    t.set_op(std::move(op));
  }
  return t;
}

#define RT_REDUCE_OP(fname, KIND)                                                                 \
  template <class B>                                                                              \
  Tensor<B> fname(const Tensor<B>& x, std::optional<size_t> axis) {                               \
    St<B> out = B::fname(x.data(), axis);                                                         \
    bool rg = x.requires_grad();                                                                  \
    return Tensor<B>::new_with_op(std::move(out), rg,                                             \
                                  rg ? std::optional<OpType>(OpType::with_axis(OpType::KIND, axis)) \
                                     : std::nullopt,                                              \
                                  {x});                                                           \
  }
RT_REDUCE_OP(mean, Mean)            // src/ops/mod.rs:614-632
RT_REDUCE_OP(max, Max)              // src/ops/mod.rs:885-903
RT_REDUCE_OP(min, Min)              // src/ops/mod.rs:907-925
RT_REDUCE_OP(prod, Prod)            // src/ops/mod.rs:929-947
RT_REDUCE_OP(logsumexp, LogSumExp)  // src/ops/mod.rs:952-970
#undef RT_REDUCE_OP

// src/ops/mod.rs:635-672.  The reference builds the global sum from a host
// float (sum_all + from_vec(&[])); B::sum_all_scalar returns that 0-D storage.
template <class B>
Tensor<B> sum(const Tensor<B>& x, std::optional<size_t> axis) {
  bool rg = x.requires_grad();
  St<B> out = axis ? B::sum_along_axis(x.data(), *axis) : B::sum_all_scalar(x.data());
  return Tensor<B>::new_with_op(
      std::move(out), rg, rg ? std::optional<OpType>(OpType::with_axis(OpType::Sum, axis)) : std::nullopt,
      {x});
}

// src/ops/mod.rs:780-798
template <class B>
Tensor<B> div_scalar(const Tensor<B>& x, float s) {
  St<B> out = B::div_scalar(x.data(), s);
  if (x.requires_grad())
    throw Error::invalid_op("Backward pass for div_scalar operation not implemented yet");
  return Tensor<B>(std::move(out), false);
}

// src/ops/mod.rs:801-824
template <class B>
Tensor<B> mul_scalar(const Tensor<B>& x, float s) {
  St<B> out = B::mul_scalar(x.data(), s);
  bool rg = x.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::MulScalar);
    ot.scalar = s;
    t.set_op(Op<B>(ot, {x}, [](const Op<B>& op, const St<B>& g) {
      return Grads<B>{B::mul_scalar(g, op.op_type.scalar)};
    }));
  }
  return t;
}

// src/ops/mod.rs:827-845
template <class B>
Tensor<B> broadcast_to(const Tensor<B>& x, const Shape& shape) {
  St<B> out = B::broadcast_to(x.data(), shape);
  bool rg = x.requires_grad();
  return Tensor<B>::new_with_op(std::move(out), rg,
                                rg ? std::optional<OpType>(OpType(OpType::Broadcast)) : std::nullopt, {x});
}

// src/ops/mod.rs:849-881
template <class B>
Tensor<B> view(const Tensor<B>& x, const Shape& shape) {
  if (shape_numel(x.shape()) != shape_numel(shape)) throw Error::incompatible("view", x.shape(), shape);
  St<B> out = x.data();
  B::set_shape(out, shape);
  bool rg = x.requires_grad();
  return Tensor<B>::new_with_op(std::move(out), rg,
                                rg ? std::optional<OpType>(OpType(OpType::View)) : std::nullopt, {x});
}

// src/ops/mod.rs:975-996 (not differentiable)
template <class B>
Tensor<B> argmax(const Tensor<B>& x, size_t axis) { return Tensor<B>(B::argmax(x.data(), axis), false); }
template <class B>
Tensor<B> argmin(const Tensor<B>& x, size_t axis) { return Tensor<B>(B::argmin(x.data(), axis), false); }

// src/ops/mod.rs:1273-1331 and equal (src/ops/mod.rs:1232-1270 family): comparisons give 1.0 / 0.0, broadcast like the
// arithmetic ops and are not differentiable.
#define RT_COMPARE_OP(fname)                                                                  \
  template <class B>                                                                          \
  Tensor<B> fname(const Tensor<B>& a, const Tensor<B>& b) { return Tensor<B>(B::fname(a.data(), b.data()), false); }
RT_COMPARE_OP(equal)
RT_COMPARE_OP(not_equal)
RT_COMPARE_OP(greater)
RT_COMPARE_OP(greater_equal)
RT_COMPARE_OP(less)
RT_COMPARE_OP(less_equal)
#undef RT_COMPARE_OP

// src/ops/mod.rs:1148-1158
template <class B>
Tensor<B> powf_scalar(const Tensor<B>& a, float b) {
  Tensor<B> bt(B::from_vec({b}, Shape{1}), false);
  return powf(a, bt);
}

// src/ops/mod.rs:1427-1447
template <class B>
Tensor<B> transpose(const Tensor<B>& x) {
  St<B> out = B::transpose(x.data());
  bool rg = x.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg)
    t.set_op(Op<B>(OpType(OpType::Transpose), {x},
                   [](const Op<B>&, const St<B>& g) { return Grads<B>{B::transpose(g)}; }));
  return t;
}

// src/ops/mod.rs:1477-1544
template <class B>
Tensor<B> concat(const std::vector<Tensor<B>>& tensors, size_t axis) {
  if (tensors.empty()) throw Error::invalid_op("Cannot concat empty list of tensors");
  Shape first = tensors[0].shape();
  if (axis >= first.size()) throw Error::invalid_index(axis);
  for (size_t i = 1; i < tensors.size(); ++i) {
    Shape s = tensors[i].shape();
    if (s.size() != first.size()) throw Error::incompatible("concat", first, s);
    for (size_t d = 0; d < s.size(); ++d)
      if (d != axis && s[d] != first[d])
        throw Error::incompatible("concat dim " + std::to_string(d) + " of tensor " + std::to_string(i), first, s);
  }
  std::vector<const St<B>*> refs;
  for (auto& t : tensors) refs.push_back(&t.data());
  St<B> out = B::concat(refs, axis);
  bool rg = false;
  for (auto& t : tensors) rg = rg || t.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Concat);
    ot.axis = axis;
    for (auto& x : tensors) ot.input_shapes.push_back(x.shape());
    t.set_op(Op<B>(ot, tensors, [](const Op<B>& op, const St<B>& g) { return B::concat_backward(op, g); }));
  }
  return t;
}

// src/ops/mod.rs:1573-1615
template <class B>
Tensor<B> slice(const Tensor<B>& input, const std::vector<Range>& ranges) {
  Shape s = input.shape();
  if (ranges.size() != s.size())
    throw Error::invalid_op("Slice ranges length " + std::to_string(ranges.size()) +
                            " must match input dimensionality " + std::to_string(s.size()));
  for (size_t i = 0; i < ranges.size(); ++i) {
    if (ranges[i].start > ranges[i].end)
      throw Error::invalid_op("Invalid slice range at dimension " + std::to_string(i));
    if (ranges[i].end > s[i]) throw Error::invalid_index(i);
  }
  St<B> out = B::slice(input.data(), ranges);
  bool rg = input.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Slice);
    ot.input_shape = s;
    ot.ranges = ranges;
    t.set_op(Op<B>(ot, {input}, [](const Op<B>& op, const St<B>& g) { return Grads<B>{B::slice_backward(op, g)}; }));
  }
  return t;
}

// src/ops/mod.rs:1642-1662
template <class B>
Tensor<B> expand_dims(const Tensor<B>& input, size_t axis) {
  if (axis > input.shape().size()) throw Error::invalid_index(axis);
  St<B> out = B::expand_dims(input.data(), axis);
  bool rg = input.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::ExpandDims);
    ot.axis = axis;
    t.set_op(Op<B>(ot, {input}, [](const Op<B>& op, const St<B>& g) { return Grads<B>{B::expand_dims_backward(op, g)}; }));
  }
  return t;
}

// src/ops/mod.rs:1689-1721
template <class B>
Tensor<B> squeeze(const Tensor<B>& input, std::optional<size_t> axis) {
  Shape orig = input.shape();
  if (axis) {
    if (*axis >= orig.size()) throw Error::invalid_index(*axis);
    if (orig[*axis] != 1)
      throw Error::invalid_op("Cannot squeeze axis " + std::to_string(*axis) + " of shape " + shape_str(orig) +
                              " (not size 1)");
  }
  St<B> out = B::squeeze(input.data(), axis);
  bool rg = input.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Squeeze);
    ot.axis = axis;
    ot.input_shape = orig;
    t.set_op(Op<B>(ot, {input}, [](const Op<B>& op, const St<B>& g) { return Grads<B>{B::squeeze_backward(op, g)}; }));
  }
  return t;
}

// src/ops/mod.rs:1781-1801
template <class B>
Tensor<B> clip(const Tensor<B>& input, float min_val, float max_val) {
  if (min_val > max_val) throw Error::invalid_op("Clip min_val cannot be greater than max_val");
  St<B> out = B::clip(input.data(), min_val, max_val);
  bool rg = input.requires_grad();
  Tensor<B> t(std::move(out), rg);
  if (rg) {
    OpType ot(OpType::Clip);
    ot.min_val = min_val;
    ot.max_val = max_val;
    t.set_op(Op<B>(ot, {input}, [](const Op<B>& op, const St<B>& g) { return Grads<B>{B::clip_backward(op, g)}; }));
  }
  return t;
}

template <class B>
Tensor<B> apply_reduction(const Tensor<B>& t, Reduction r) {
  switch (r) {
    case Reduction::None: return t;
    case Reduction::Sum: return sum(t, std::nullopt);
    default: return mean(t, std::nullopt);
  }
}

// src/ops/mod.rs:553-595: sub -> mul(diff, diff) -> reduction
template <class B>
Tensor<B> mse_loss(const Tensor<B>& preds, const Tensor<B>& targets, Reduction r) {
  if (preds.shape() != targets.shape()) throw Error::incompatible("mse_loss", preds.shape(), targets.shape());
  Tensor<B> diff = sub(preds, targets);
  Tensor<B> sq = mul(diff, diff);
  return apply_reduction(sq, r);
}

// src/ops/mod.rs:1057-1113
template <class B>
Tensor<B> binary_cross_entropy_with_logits(const Tensor<B>& logits, const Tensor<B>& targets, Reduction r) {
  if (logits.shape() != targets.shape())
    throw Error::incompatible("binary_cross_entropy_with_logits", logits.shape(), targets.shape());
  Tensor<B> minus_one = Tensor<B>::from_vec({-1.0f}, Shape{}, false);
  Tensor<B> one = Tensor<B>::from_vec({1.0f}, Shape{}, false);
  Tensor<B> term1 = relu(logits);
  Tensor<B> term2 = mul(logits, targets);
  Tensor<B> abs_l = abs(logits);
  Tensor<B> neg_abs = mul(abs_l, minus_one);
  Tensor<B> e = exp(neg_abs);
  Tensor<B> one_plus = add(one, e);
  Tensor<B> term3 = ln(one_plus);
  Tensor<B> inter = sub(term1, term2);
  Tensor<B> elems = add(inter, term3);
  return apply_reduction(elems, r);
}

// src/ops/mod.rs:1356-1424: log_softmax -> mul(one-hot) -> sum(axis) -> mul(-1) -> reduction
template <class B>
Tensor<B> softmax_cross_entropy(const Tensor<B>& logits, const Tensor<B>& targets, size_t axis, Reduction r) {
  if (logits.shape() != targets.shape())
    throw Error::incompatible("softmax_cross_entropy", logits.shape(), targets.shape());
  if (axis >= logits.shape().size()) throw Error::invalid_index(axis);
  Tensor<B> log_probs = log_softmax(logits, axis);
  Tensor<B> prod = mul(log_probs, targets);
  Tensor<B> s = sum(prod, axis);
  Tensor<B> minus_one = Tensor<B>::from_vec({-1.0f}, Shape{}, false);
  Tensor<B> per_sample = mul(s, minus_one);
  return apply_reduction(per_sample, r);
}

// ---- fused forward ops (not in the reference) -----------------------------------------------------------------------
// They sit beside the unchanged ops and compute exactly what the corresponding chain of reference ops computes.  A
// backend that has no fused kernels (the CPU restatement used by the tests) gets the chain itself.
template <class B, class = void>
struct HasFusedForward : std::false_type {};
template <class B>
struct HasFusedForward<B, std::void_t<decltype(&B::relu_max_pool2d)>> : std::true_type {};

// max_pool2d(relu(x)): one kernel forward (relu(x) is never materialised), one backward.
template <class B>
Tensor<B> fused_relu_max_pool2d(const Tensor<B>& input, Pair kernel, Pair stride, Pair padding) {
  if constexpr (!HasFusedForward<B>::value) {
    return max_pool2d(relu(input), kernel, stride, padding);
  } else {
    auto r = B::relu_max_pool2d(input.data(), kernel, stride, padding);
    bool rg = input.requires_grad();
    Tensor<B> t(std::move(r.first), rg);
    if (rg) {
      Tensor<B> idx(std::move(r.second), false);
      OpType ot(OpType::FusedReluMaxPool2D);
      ot.kernel_size = kernel;
      ot.stride = stride;
      ot.padding = padding;
      t.set_op(Op<B>(ot, {input, idx}, [](const Op<B>& op, const St<B>& g) {
        St<B> gi = B::relu_max_pool2d_backward(op, g);
        return Grads<B>{std::move(gi), B::unused_grad(B::shape(op.inputs[1].data()))};
      }));
    }
    return t;
  }
}

// max_pool2d(relu(conv2d(x, w, bias)), 2x2, stride 2): the head of a CNN block as the reference's example spells it with three
// ops (examples/train_mnist_cnn_cpu.rs:216-233).  The convolution output is never kept: the backward pass gets the gradient of
// the convolution output from the pooled values (y > 0 exactly where the winning input was positive) and the saved indices.
template <class B>
Tensor<B> fused_conv2d_relu_max_pool2d(const Tensor<B>& input, const Tensor<B>& weights, const Tensor<B>* bias, Pair stride,
                                       Pair padding) {
  if constexpr (!HasFusedForward<B>::value) {
    return max_pool2d(relu(conv2d(input, weights, bias, stride, padding)), {2, 2}, {2, 2}, {0, 0});
  } else {
    auto r = B::conv2d_relu_max_pool2x2(input.data(), weights.data(), bias ? &bias->data() : nullptr, stride, padding);
    bool rg = input.requires_grad() || weights.requires_grad() || (bias && bias->requires_grad());
    Tensor<B> t(r.first, rg);  // shares the buffer with the saved copy below (buffers are immutable)
    if (rg) {
      OpType ot(OpType::FusedConvReluMaxPool2D);
      ot.stride = stride;
      ot.padding = padding;
      ot.kernel_size = {2, 2};
      Tensor<B> b = bias ? *bias : Tensor<B>(B::zeros(Shape{weights.shape()[0]}), false);
      Tensor<B> y_saved(std::move(r.first), false), idx(std::move(r.second), false);
      t.set_op(Op<B>(ot, {input, weights, b, y_saved, idx}, [](const Op<B>& op, const St<B>& g) {
        auto gr = B::conv2d_relu_max_pool2x2_backward(op.inputs[0].data(), op.inputs[1].data(), op.inputs[3].data(), op.inputs[4].data(), g,
                                                      op.op_type.stride, op.op_type.padding, op.inputs[0].requires_grad(),
                                                      op.inputs[1].requires_grad(), op.inputs[2].requires_grad());
        St<B> gb = std::get<2>(gr) ? std::move(*std::get<2>(gr)) : B::zeros(Shape{0});
        return Grads<B>{std::move(std::get<0>(gr)), std::move(std::get<1>(gr)), std::move(gb), B::unused_grad(B::shape(op.inputs[3].data())),
                        B::unused_grad(B::shape(op.inputs[4].data()))};
      }));
    }
    return t;
  }
}

// concat({slice(x, rows r0..r1, all columns), h}, axis 1) for a 2-D x that needs no gradient: what a recurrent model does at every
// timestep with its time-major input (examples/lstm_char_rnn_cpu.rs).  The row slice is never materialised.
template <class B>
Tensor<B> fused_rows_concat(const Tensor<B>& x, size_t r0, size_t r1, const Tensor<B>& h) {
  if constexpr (!HasFusedForward<B>::value) {
    return concat<B>({slice(x, {{r0, r1}, {0, x.shape().at(1)}}), h}, 1);
  } else {
    if (x.requires_grad()) return concat<B>({slice(x, {{r0, r1}, {0, x.shape().at(1)}}), h}, 1);
    St<B> out = B::concat_rows_with(x.data(), r0, r1, h.data());
    bool rg = h.requires_grad();
    Tensor<B> t(std::move(out), rg);
    if (rg) {
      OpType ot(OpType::Concat);  // the backward of a concatenation whose first input takes no gradient
      ot.axis = 1;
      Tensor<B> left(B::unused_grad(Shape{r1 - r0, x.shape()[1]}), false);
      ot.input_shapes = {left.shape(), h.shape()};
      t.set_op(Op<B>(ot, {left, h}, [](const Op<B>& op, const St<B>& g) { return B::concat_backward(op, g); }));
    }
    return t;
  }
}

// -mean over the rows of sum_k targets * log_softmax(logits, 1): the loss of the reference's classification examples
// (examples/train_mnist_cpu.rs:63-97: log_softmax -> mul -> sum(axis 1) -> mean -> mul(-1)), 2-D logits.
template <class B>
Tensor<B> fused_softmax_nll(const Tensor<B>& logits, const Tensor<B>& targets) {
  if (logits.shape() != targets.shape()) throw Error::incompatible("fused_softmax_nll", logits.shape(), targets.shape());
  if (logits.shape().size() != 2) throw Error::invalid_op("fused_softmax_nll expects [rows, classes] logits");
  if constexpr (!HasFusedForward<B>::value) {
    Tensor<B> e = mul(log_softmax(logits, 1), targets);
    Tensor<B> per = sum(e, 1);
    Tensor<B> m = mean(per, std::nullopt);
    Tensor<B> minus_one = Tensor<B>::from_vec({-1.0f}, Shape{}, false);
    return mul(m, minus_one);
  } else {
    St<B> out = B::softmax_nll(logits.data(), targets.data());
    bool rg = logits.requires_grad() || targets.requires_grad();
    Tensor<B> t(std::move(out), rg);
    if (rg) {
      t.set_op(Op<B>(OpType(OpType::FusedSoftmaxNll), {logits, targets}, [](const Op<B>& op, const St<B>& g) {
        auto p = B::softmax_nll_backward(op, g);
        return Grads<B>{std::move(p.first), std::move(p.second)};
      }));
    }
    return t;
  }
}

// LSTM cell update from the pre-activation gates [B, 4H] (column blocks: input, forget, candidate, output), as the
// reference's char-LSTM example spells it with slices (examples/lstm_char_rnn_cpu.rs):
//   c = sigmoid(f) * c_prev + sigmoid(i) * tanh(g)
template <class B>
Tensor<B> fused_lstm_cell_c(const Tensor<B>& gates, const Tensor<B>& c_prev) {
  const Shape& gs = gates.shape();
  if (gs.size() != 2 || c_prev.shape().size() != 2 || gs[0] != c_prev.shape()[0] || gs[1] != 4 * c_prev.shape()[1])
    throw Error::incompatible("fused_lstm_cell_c", gs, c_prev.shape());
  const size_t Bn = gs[0], H = c_prev.shape()[1];
  if constexpr (!HasFusedForward<B>::value) {
    Tensor<B> ig = sigmoid(slice(gates, {{0, Bn}, {0, H}}));
    Tensor<B> fg = sigmoid(slice(gates, {{0, Bn}, {H, 2 * H}}));
    Tensor<B> gg = tanh(slice(gates, {{0, Bn}, {2 * H, 3 * H}}));
    return add(mul(fg, c_prev), mul(ig, gg));
  } else {
    St<B> out = B::lstm_cell_c(gates.data(), c_prev.data());
    bool rg = gates.requires_grad() || c_prev.requires_grad();
    Tensor<B> t(std::move(out), rg);
    if (rg) {
      t.set_op(Op<B>(OpType(OpType::FusedLstmCellC), {gates, c_prev}, [](const Op<B>& op, const St<B>& g) {
        auto p = B::lstm_cell_c_backward(op, g);
        return Grads<B>{std::move(p.first), std::move(p.second)};
      }));
    }
    return t;
  }
}

//   h = sigmoid(o) * tanh(c)
template <class B>
Tensor<B> fused_lstm_cell_h(const Tensor<B>& gates, const Tensor<B>& c) {
  const Shape& gs = gates.shape();
  if (gs.size() != 2 || c.shape().size() != 2 || gs[0] != c.shape()[0] || gs[1] != 4 * c.shape()[1])
    throw Error::incompatible("fused_lstm_cell_h", gs, c.shape());
  const size_t Bn = gs[0], H = c.shape()[1];
  if constexpr (!HasFusedForward<B>::value) {
    Tensor<B> og = sigmoid(slice(gates, {{0, Bn}, {3 * H, 4 * H}}));
    return mul(og, tanh(c));
  } else {
    St<B> out = B::lstm_cell_h(gates.data(), c.data());
    bool rg = gates.requires_grad() || c.requires_grad();
    Tensor<B> t(std::move(out), rg);
    if (rg) {
      t.set_op(Op<B>(OpType(OpType::FusedLstmCellH), {gates, c}, [](const Op<B>& op, const St<B>& g) {
        auto p = B::lstm_cell_h_backward(op, g);
        return Grads<B>{std::move(p.first), std::move(p.second)};
      }));
    }
    return t;
  }
}

}  // namespace ops

template <class B>
Tensor<B> Tensor<B>::view(const Shape& s) const { return ops::view(*this, s); }
template <class B>
Tensor<B> Tensor<B>::broadcast_to(const Shape& s) const { return ops::broadcast_to(*this, s); }

// =============================================================================
// Optimizers (src/optim.rs).  Parameters without a gradient, or whose gradient
// shape differs from the data shape, are skipped.
// =============================================================================
// src/data.rs:125-209.  The reference copies x and y to the host, picks `batch_size` distinct random rows there and
// uploads the two batches; here the rows are gathered by the backend (on the device for the CUDA backend) and only the
// indices are chosen on the host.  get_batch takes the indices, get_random_batch samples them without replacement
// (rand::seq::index::sample in the reference; a partial Fisher-Yates shuffle of a seeded generator here).
namespace data {

template <class B>
std::pair<Tensor<B>, Tensor<B>> get_batch(const Tensor<B>& x, const Tensor<B>& y, const std::vector<size_t>& indices) {
  const Shape xs = x.shape(), ys = y.shape();
  if (xs.empty() || xs[0] == 0) throw Error(ErrorKind::EmptyTensor, "Cannot perform operation on empty tensor");
  if (ys.empty() || ys[0] == 0) throw Error(ErrorKind::EmptyTensor, "Cannot perform operation on empty tensor");
  const size_t n = xs[0];
  if (ys[0] != n) throw Error::shape_mismatch(Shape{n}, Shape{ys[0]});
  if (indices.empty()) throw Error::invalid_op("Batch size cannot be zero");
  if (indices.size() > n) throw Error(ErrorKind::DimensionMismatch, "batch size exceeds the number of samples");
  const size_t fx = xs.size() > 1 ? xs[1] : 1, fy = ys.size() > 1 ? ys[1] : 1;  // as the reference: 1 if 1-D
  return {Tensor<B>(B::gather_rows(x.data(), n, fx, indices), false), Tensor<B>(B::gather_rows(y.data(), n, fy, indices), false)};
}

inline std::vector<size_t> sample_indices(size_t n, size_t k, uint64_t seed) {
  std::vector<size_t> pool(n);
  for (size_t i = 0; i < n; ++i) pool[i] = i;
  uint64_t s = seed;
  auto next = [&]() {  // splitmix64
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  };
  for (size_t i = 0; i < k; ++i) std::swap(pool[i], pool[i + (size_t)(next() % (n - i))]);
  pool.resize(k);
  return pool;
}

template <class B>
std::pair<Tensor<B>, Tensor<B>> get_random_batch(const Tensor<B>& x, const Tensor<B>& y, size_t batch_size, uint64_t seed) {
  const Shape xs = x.shape();
  if (xs.empty() || xs[0] == 0) throw Error(ErrorKind::EmptyTensor, "Cannot perform operation on empty tensor");
  if (batch_size == 0) throw Error::invalid_op("Batch size cannot be zero");
  if (batch_size > xs[0]) throw Error(ErrorKind::DimensionMismatch, "batch size exceeds the number of samples");
  return get_batch(x, y, sample_indices(xs[0], batch_size, seed));
}

}  // namespace data

namespace optim {

template <class B>
std::vector<std::pair<size_t, typename B::Storage>> collect_updates(const std::vector<Tensor<B>>& params) {
  std::vector<std::pair<size_t, typename B::Storage>> ups;
  for (size_t i = 0; i < params.size(); ++i) {
    const auto& p = params[i];
    if (!p.requires_grad() || !p.grad()) continue;
    if (B::shape(*p.grad()) != p.shape()) continue;
    ups.emplace_back(i, *p.grad());
  }
  return ups;
}

template <class B>
void zero_grad_all(const std::vector<Tensor<B>>& params) {
  for (auto& p : params)
    if (p.requires_grad()) p.zero_grad();
}

// src/optim.rs:10-83
template <class B>
struct Sgd {
  std::vector<Tensor<B>> parameters;
  float learning_rate;
  Sgd(std::vector<Tensor<B>> p, float lr) : parameters(std::move(p)), learning_rate(lr) {}
  void step() {
    for (auto& u : collect_updates(parameters))
      B::sgd_step(parameters[u.first].data_mut(), u.second, learning_rate);
  }
  void zero_grad() { zero_grad_all(parameters); }
};

// src/optim.rs:87-191 (t is incremented before the parameter loop)
template <class B>
struct Adam {
  std::vector<Tensor<B>> parameters;
  float learning_rate, beta1, beta2, epsilon;
  std::vector<typename B::Storage> m_states, v_states;
  size_t t = 0;
  Adam(std::vector<Tensor<B>> p, float lr, float b1, float b2, float eps)
      : parameters(std::move(p)), learning_rate(lr), beta1(b1), beta2(b2), epsilon(eps) {
    for (auto& x : parameters) {
      m_states.push_back(B::zeros(x.shape()));
      v_states.push_back(B::zeros(x.shape()));
    }
  }
  void step() {
    t += 1;
    for (auto& u : collect_updates(parameters))
      B::adam_step(parameters[u.first].data_mut(), u.second, m_states[u.first], v_states[u.first],
                   learning_rate, beta1, beta2, epsilon, t);
  }
  void zero_grad() { zero_grad_all(parameters); }
};

// src/optim.rs:197-271
template <class B>
struct MomentumSGD {
  std::vector<Tensor<B>> parameters;
  float learning_rate, momentum;
  std::vector<typename B::Storage> velocities;
  MomentumSGD(std::vector<Tensor<B>> p, float lr, float mu)
      : parameters(std::move(p)), learning_rate(lr), momentum(mu) {
    for (auto& x : parameters) velocities.push_back(B::zeros(x.shape()));
  }
  void step() {
    for (auto& u : collect_updates(parameters))
      B::momentum_sgd_step(parameters[u.first].data_mut(), u.second, velocities[u.first], learning_rate,
                           momentum);
  }
  void zero_grad() { zero_grad_all(parameters); }
};

// src/optim.rs:278-368
template <class B>
struct AdaGrad {
  std::vector<Tensor<B>> parameters;
  float learning_rate, epsilon;
  std::vector<typename B::Storage> accumulated_sq_grad;
  AdaGrad(std::vector<Tensor<B>> p, float lr, float eps)
      : parameters(std::move(p)), learning_rate(lr), epsilon(eps) {
    for (auto& x : parameters) accumulated_sq_grad.push_back(B::zeros(x.shape()));
  }
  void step() {
    for (auto& u : collect_updates(parameters))
      B::adagrad_step(parameters[u.first].data_mut(), u.second, accumulated_sq_grad[u.first], learning_rate,
                      epsilon);
  }
  void zero_grad() { zero_grad_all(parameters); }
};

}  // namespace optim

// =============================================================================
// Finite-difference gradient checker (src/test_utils.rs:17-265).
// =============================================================================
struct GradCheckResult {
  bool ok;
  float max_rel_error, max_abs_error;
  size_t at_index;
  std::vector<float> analytical, numerical;
};

// src/test_utils.rs:221-265: per element abs/max(|a|,|n|) when both exceed 1e-8,
// else the absolute error; gate on the maximum.
inline GradCheckResult compare_gradients(const std::vector<float>& a, const std::vector<float>& n, float tol) {
  GradCheckResult r{true, 0.f, 0.f, 0, a, n};
  if (a.size() != n.size()) throw Error::internal("Gradient size mismatch");
  for (size_t i = 0; i < a.size(); ++i) {
    float abs_err = std::fabs(a[i] - n[i]);
    float rel = (std::fabs(a[i]) > 1e-8f && std::fabs(n[i]) > 1e-8f)
                    ? abs_err / std::max(std::fabs(a[i]), std::fabs(n[i]))
                    : abs_err;
    if (rel > r.max_rel_error) {
      r.max_rel_error = rel;
      r.max_abs_error = abs_err;
      r.at_index = i;
    }
  }
  r.ok = r.max_rel_error <= tol;
  return r;
}

template <class B, class F>
GradCheckResult check_gradient(F func, std::vector<Tensor<B>> inputs, size_t idx, float epsilon, float tol) {
  if (idx >= inputs.size()) throw Error::invalid_op("input_idx_to_check is out of bounds");
  const Tensor<B>& target = inputs[idx];
  if (!target.requires_grad()) return GradCheckResult{true, 0, 0, 0, {}, {}};
  // analytical (src/test_utils.rs:63-127)
  for (auto& t : inputs)
    if (t.requires_grad()) t.zero_grad();
  Tensor<B> loss = func(inputs);
  if (shape_numel(loss.shape()) != 1)
    throw Error::invalid_op("Function must return a scalar tensor for gradient checking");
  loss.backward();
  std::vector<float> analytical =
      target.grad() ? B::copy_to_host(*target.grad()) : std::vector<float>(std::max<size_t>(target.size(), 1), 0.f);
  // numerical (src/test_utils.rs:129-219)
  std::vector<float> orig = B::copy_to_host(target.data());
  size_t n = std::max<size_t>(target.size(), 1);
  std::vector<float> numerical(n, 0.f);
  for (size_t i = 0; i < n; ++i) {
    auto eval = [&](float delta) {
      std::vector<float> d = orig;
      d[i] += delta;
      std::vector<Tensor<B>> in2 = inputs;
      in2[idx] = Tensor<B>(B::from_vec(std::move(d), target.shape()), target.requires_grad());
      Tensor<B> l = func(in2);
      return B::copy_to_host(l.data()).at(0);
    };
    float lp = eval(epsilon), lm = eval(-epsilon);
    numerical[i] = (lp - lm) / (2.0f * epsilon);
  }
  return compare_gradients(analytical, numerical, tol);
}

}  // namespace rt
