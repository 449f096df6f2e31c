// `B200Backend`: the Backend implementation that forwards every trait method of the
// reference (src/backend/mod.rs:14-656) to one C-ABI entry point of librt_b200.so
// (include/rt_b200.h).  This is the C++ twin of the Rust shim a maintainer would write
// as `impl Backend for B200Backend`; it owns no math, only shape bookkeeping (integer,
// host side) and device-buffer lifetime.
//
// Storage is a reference-counted device buffer plus a shape.  Buffers are immutable once
// produced by an op, so copying a Storage is O(1) yet indistinguishable from the deep
// copy the reference's `Clone` performs; the in-place mutators (optimizer steps,
// update_from_host) first make the buffer unique.
#pragma once
#include <memory>
#include <cmath>
#include <optional>
#include <random>
#include <tuple>
#include <vector>

#include "../../../include/rt_b200.h"
#include "autograd.hpp"

namespace rt {

struct DeviceBuffer {
  rt_ctx* ctx;
  float* ptr;
  size_t numel;
  DeviceBuffer(rt_ctx* c, float* p, size_t n) : ctx(c), ptr(p), numel(n) {}
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  ~DeviceBuffer() {
    if (ptr) rt_free(ctx, ptr);
  }
};

struct DeviceStorage {
  std::shared_ptr<DeviceBuffer> buf;
  Shape shape;
  float* ptr() const { return buf ? buf->ptr : nullptr; }
  size_t numel() const { return shape_numel(shape); }
};

struct B200Backend {
  using Storage = DeviceStorage;
  using OpB = Op<B200Backend>;

  static rt_ctx*& ctx_slot() {
    static rt_ctx* c = nullptr;
    return c;
  }
  static rt_ctx* ctx() {
    if (!ctx_slot()) throw Error(ErrorKind::CudaError, "B200Backend: no context (call rth_init first)");
    return ctx_slot();
  }
  static void check(rt_status st) {
    if (st != RT_OK) throw Error((ErrorKind)st, rt_last_error(ctx_slot()));
  }
  static std::vector<int64_t> dims(const Shape& s) { return std::vector<int64_t>(s.begin(), s.end()); }

  static Storage alloc(const Shape& s) {
    size_t n = shape_numel(s);
    void* p = nullptr;
    check(rt_malloc(ctx(), sizeof(float) * std::max<size_t>(n, 1), &p));
    return Storage{std::make_shared<DeviceBuffer>(ctx(), (float*)p, n), s};
  }
  static void make_unique(Storage& s) {
    if (s.buf && s.buf.use_count() > 1) {
      Storage c = alloc(s.shape);
      check(rt_memcpy_d2d(ctx(), c.ptr(), s.ptr(), sizeof(float) * s.numel()));
      s.buf = std::move(c.buf);
    }
  }

  // ---- factories / access (mod.rs:44-88, 248-252) --------------------------------------
  static Storage filled(const Shape& s, float v) {
    Storage r = alloc(s);
    check(rt_fill(ctx(), r.ptr(), v, (int64_t)r.numel()));
    return r;
  }
  static Storage zeros(const Shape& s) { return filled(s, 0.f); }
  static Storage ones(const Shape& s) { return filled(s, 1.f); }
  static Storage from_vec(std::vector<float> v, const Shape& s) {
    if (v.size() != shape_numel(s)) throw Error::shape_mismatch(s, Shape{v.size()});
    if (v.size() == 1) return filled(s, v[0]);  // a constant: no host copy, safe inside graph capture
    Storage r = alloc(s);
    check(rt_memcpy_h2d(ctx(), r.ptr(), v.data(), sizeof(float) * v.size()));
    return r;
  }
  // ---- random factories (mod.rs:57-69; src/backend/cpu.rs:133-194; src/init.rs:7-52) ------------------------
  // The generator state is (seed, counter offset); manual_seed restarts the stream.  Without a seed the first use
  // takes one from the operating system, like rand's thread-local generator.
  struct RngState { uint64_t seed = 0, offset = 0; bool seeded = false; };
  static RngState& rng() {
    static RngState s;
    return s;
  }
  static void manual_seed(uint64_t seed) { rng() = RngState{seed, 0, true}; }
  static RngState& rng_ready() {
    RngState& s = rng();
    if (!s.seeded) {
      std::random_device rd;
      s = RngState{((uint64_t)rd() << 32) ^ rd(), 0, true};
    }
    return s;
  }
  static Storage random_uniform(const Shape& shape, float low, float high) {
    if (shape_numel(shape) == 0) return zeros(shape);
    RngState& s = rng_ready();
    Storage r = alloc(shape);
    check(rt_random_uniform(ctx(), r.ptr(), (int64_t)r.numel(), low, high, s.seed, s.offset));
    s.offset += (r.numel() + 3) / 4;
    return r;
  }
  static Storage random_normal(const Shape& shape, float mean, float std_dev) {
    if (shape_numel(shape) == 0) return zeros(shape);
    RngState& s = rng_ready();
    Storage r = alloc(shape);
    check(rt_random_normal(ctx(), r.ptr(), (int64_t)r.numel(), mean, std_dev, s.seed, s.offset));
    s.offset += (r.numel() + 3) / 4;
    return r;
  }
  static Storage bernoulli(const Shape& shape, float p) {
    if (shape_numel(shape) == 0) return zeros(shape);
    RngState& s = rng_ready();
    Storage r = alloc(shape);
    check(rt_bernoulli(ctx(), r.ptr(), (int64_t)r.numel(), p, s.seed, s.offset));
    s.offset += (r.numel() + 3) / 4;
    return r;
  }
  static Storage kaiming_uniform(size_t fan_in, const Shape& shape) {  // src/init.rs:7-52
    if (shape.empty()) throw Error::invalid_op("Cannot initialize tensor with empty shape");
    if (shape_numel(shape) == 0) return zeros(shape);
    if (fan_in == 0) throw Error::invalid_op("Fan-in cannot be zero for Kaiming initialization");
    const float bound = std::sqrt(6.0f / (float)fan_in);
    return random_uniform(shape, -bound, bound);
  }
  // Rows idx[i] of x viewed as [rows, row_len] -> [idx.size(), row_len] (the gather of data::get_random_batch on the
  // device: only the indices travel).  Indices are checked on the host.
  static Storage gather_rows(const Storage& x, size_t rows, size_t row_len, const std::vector<size_t>& idx) {
    std::vector<int32_t> h(idx.size());
    for (size_t i = 0; i < idx.size(); ++i) {
      if (idx[i] >= rows) throw Error(ErrorKind::InvalidIndex, "gather_rows: index out of range");
      h[i] = (int32_t)idx[i];
    }
    Storage out = alloc(Shape{idx.size(), row_len});
    if (idx.empty() || row_len == 0) return out;
    void* d = nullptr;
    check(rt_malloc(ctx(), sizeof(int32_t) * h.size(), &d));
    rt_status st = rt_memcpy_h2d(ctx(), d, h.data(), sizeof(int32_t) * h.size());
    if (st == RT_OK) st = rt_gather_rows(ctx(), x.ptr(), (int64_t)rows, (int64_t)row_len, static_cast<const int32_t*>(d), (int64_t)h.size(), out.ptr());
    rt_free(ctx(), d);
    check(st);
    return out;
  }
  static const Shape& shape(const Storage& s) { return s.shape; }
  static size_t size(const Storage& s) { return s.numel(); }
  static std::vector<float> copy_to_host(const Storage& s) {
    std::vector<float> v(s.numel());
    check(rt_memcpy_d2h(ctx(), v.data(), s.ptr(), sizeof(float) * v.size()));
    return v;
  }
  static void update_from_host(Storage& s, const std::vector<float>& d) {
    if (s.numel() != d.size()) throw Error::shape_mismatch(s.shape, Shape{d.size()});
    make_unique(s);
    check(rt_memcpy_h2d(ctx(), s.ptr(), d.data(), sizeof(float) * d.size()));
  }
  static void set_data(Storage& s, Storage d) { s = std::move(d); }
  static void set_shape(Storage& s, const Shape& shape) {
    if (shape_numel(shape) != s.numel()) throw Error::shape_mismatch(shape, s.shape);
    s.shape = shape;
  }
  // Gradient slot of an input that never receives a gradient (the index tensor of
  // max_pool2d): the reference allocates zeros that are dropped unread.
  static Storage unused_grad(const Shape& s) { return Storage{nullptr, s}; }

  // ---- elementwise -----------------------------------------------------------------------
  static Storage unary(int op, const Storage& x, float p0 = 0.f, float p1 = 0.f) {
    Storage y = alloc(x.shape);
    check(rt_unary(ctx(), op, x.ptr(), y.ptr(), (int64_t)x.numel(), p0, p1));
    return y;
  }
  static Storage unary_bwd(int op, const OpB& o, const Storage& g, float p0 = 0.f, float p1 = 0.f) {
    if (o.inputs.empty()) throw Error::invalid_op("backward requires 1 input");
    const Storage& x = o.inputs[0].data();
    if (x.shape != g.shape) throw Error::shape_mismatch(x.shape, g.shape);
    Storage dx = alloc(x.shape);
    check(rt_unary_backward(ctx(), op, x.ptr(), g.ptr(), dx.ptr(), (int64_t)x.numel(), p0, p1));
    return dx;
  }
  // Broadcast shape.  For add/mul/powf/maximum/minimum/comparisons the reference takes the larger
  // extent when one side is 1 and then asks ndarray to stretch each operand, which fails when an
  // extent 0 meets an extent 1 (src/ops/cpu_ops.rs:319-352; src/util.rs:2-26); sub/div use ndarray's
  // operator broadcasting, where 1 stretches to 0 (src/backend/cpu.rs:1259-1269).
  static Shape bshape(const Shape& a, const Shape& b, const char* op, bool ndarray_operator = false) {
    size_t nd = std::max(a.size(), b.size());
    Shape out(nd);
    for (size_t i = 0; i < nd; ++i) {
      size_t ad = i < nd - a.size() ? 1 : a[i - (nd - a.size())];
      size_t bd = i < nd - b.size() ? 1 : b[i - (nd - b.size())];
      if (ad == bd) out[i] = ad;
      else if (ad == 1 || bd == 1) {
        out[i] = ndarray_operator ? (ad == 1 ? bd : ad) : std::max(ad, bd);
        if ((out[i] != ad && ad != 1) || (out[i] != bd && bd != 1)) throw Error::incompatible(op, a, b);
      } else throw Error::incompatible(op, a, b);
    }
    return out;
  }
  static bool is_operator_op(int op) { return op == RT_SUB || op == RT_DIV; }
  static Storage binary(int op, const Storage& a, const Storage& b, const char* name) {
    Storage out = alloc(bshape(a.shape, b.shape, name, is_operator_op(op)));
    auto as = dims(a.shape), bs = dims(b.shape);
    check(rt_binary(ctx(), op, a.ptr(), as.data(), (int)as.size(), b.ptr(), bs.data(), (int)bs.size(), out.ptr()));
    return out;
  }
  static std::pair<Storage, Storage> binary_bwd(int op, const OpB& o, const Storage& g, const char* name) {
    if (o.inputs.size() != 2) throw Error::invalid_op(std::string(name) + " requires 2 inputs");
    const Storage& a = o.inputs[0].data();
    const Storage& b = o.inputs[1].data();
    Shape os = bshape(a.shape, b.shape, name, is_operator_op(op));
    if (g.numel() != shape_numel(os)) throw Error::incompatible(name, os, g.shape);
    bool need_a = o.inputs[0].requires_grad(), need_b = o.inputs[1].requires_grad();
    Storage da = need_a ? alloc(a.shape) : Storage{nullptr, a.shape};
    Storage db = need_b ? alloc(b.shape) : Storage{nullptr, b.shape};
    auto as = dims(a.shape), bs = dims(b.shape);
    check(rt_binary_backward(ctx(), op, a.ptr(), as.data(), (int)as.size(), b.ptr(), bs.data(), (int)bs.size(), g.ptr(),
                             da.ptr(), db.ptr()));
    return {std::move(da), std::move(db)};
  }
  static Storage mul(const Storage& a, const Storage& b) { return binary(RT_MUL, a, b, "mul"); }
  static Storage add(const Storage& a, const Storage& b) { return binary(RT_ADD, a, b, "add"); }
  static Storage sub(const Storage& a, const Storage& b) { return binary(RT_SUB, a, b, "sub"); }
  static Storage div(const Storage& a, const Storage& b) { return binary(RT_DIV, a, b, "div"); }
  static Storage powf(const Storage& a, const Storage& b) { return binary(RT_POWF, a, b, "powf"); }
  static Storage maximum(const Storage& a, const Storage& b) { return binary(RT_MAXIMUM, a, b, "maximum"); }
  static Storage minimum(const Storage& a, const Storage& b) { return binary(RT_MINIMUM, a, b, "minimum"); }
  static Storage equal(const Storage& a, const Storage& b) { return binary(RT_EQUAL, a, b, "equal"); }
  static Storage not_equal(const Storage& a, const Storage& b) { return binary(RT_NOT_EQUAL, a, b, "not_equal"); }
  static Storage greater(const Storage& a, const Storage& b) { return binary(RT_GREATER, a, b, "greater"); }
  static Storage greater_equal(const Storage& a, const Storage& b) { return binary(RT_GREATER_EQUAL, a, b, "greater_equal"); }
  static Storage less(const Storage& a, const Storage& b) { return binary(RT_LESS, a, b, "less"); }
  static Storage less_equal(const Storage& a, const Storage& b) { return binary(RT_LESS_EQUAL, a, b, "less_equal"); }
  // true when `small` (rank <= rank of `full`, no empty axis) broadcasts onto `full` by stretching 1s only
  static bool stretches_onto(const Shape& small, const Shape& full) {
    if (small.size() > full.size()) return false;
    const size_t off = full.size() - small.size();
    for (size_t i = 0; i < small.size(); ++i)
      if (small[i] != full[i + off] && small[i] != 1) return false;
    return true;
  }
  static std::pair<Storage, Storage> mul_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_MUL, o, g, "mul"); }
  static std::pair<Storage, Storage> add_backward(const OpB& o, const Storage& g) {
    // same-shape add: both gradients are the upstream gradient itself (no copy)
    if (o.inputs.size() == 2 && o.inputs[0].data().shape == g.shape && o.inputs[1].data().shape == g.shape) return {g, g};
    // full-shape a + broadcast b (a bias): da is the upstream gradient itself, db its sum over the stretched axes
    if (o.inputs.size() == 2 && o.inputs[0].data().shape == g.shape && g.numel() > 0 && stretches_onto(o.inputs[1].data().shape, g.shape)) {
      const Shape& bs = o.inputs[1].data().shape;
      const auto& bias = o.inputs[1];
      if (bias.requires_grad() && bias.grad() && g.shape.size() == 2 && bs.size() == 1 && bs[0] == g.shape[1] && g.shape[0] <= 1024 &&
          bias.grad()->shape == bs) {
        // the bias already holds a gradient (it is used at every timestep): add this one's column sums to it in place
        Storage& acc = bias.grad_mut();
        make_unique(acc);
        check(rt_sum_rows_accumulate(ctx(), g.ptr(), (int64_t)g.shape[0], (int64_t)g.shape[1], acc.ptr()));
        return {g, unused_grad(bs)};
      }
      return {g, bias.requires_grad() ? unbroadcast(g, bs) : unused_grad(bs)};
    }
    return binary_bwd(RT_ADD, o, g, "add");
  }
  static std::pair<Storage, Storage> sub_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_SUB, o, g, "sub"); }
  static std::pair<Storage, Storage> div_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_DIV, o, g, "div"); }
  static std::pair<Storage, Storage> powf_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_POWF, o, g, "powf"); }
  static std::pair<Storage, Storage> maximum_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_MAXIMUM, o, g, "maximum"); }
  static std::pair<Storage, Storage> minimum_backward(const OpB& o, const Storage& g) { return binary_bwd(RT_MINIMUM, o, g, "minimum"); }

  static Storage div_scalar(const Storage& x, float s) {
    if (s == 0.0f) throw Error::invalid_op("Division by zero scalar");
    return unary(RT_DIV_SCALAR, x, s);
  }
  static Storage mul_scalar(const Storage& x, float s) { return unary(RT_MUL_SCALAR, x, s); }
  static Storage exp(const Storage& x) { return unary(RT_EXP, x); }
  static Storage ln(const Storage& x) { return unary(RT_LN, x); }
  static Storage abs(const Storage& x) { return unary(RT_ABS, x); }
  static Storage tanh(const Storage& x) { return unary(RT_TANH, x); }
  static Storage sin(const Storage& x) { return unary(RT_SIN, x); }
  static Storage cos(const Storage& x) { return unary(RT_COS, x); }
  static Storage tan(const Storage& x) { return unary(RT_TAN, x); }
  static Storage relu(const Storage& x) { return unary(RT_RELU, x); }
  static Storage sigmoid(const Storage& x) { return unary(RT_SIGMOID, x); }
  static Storage softplus(const Storage& x) { return unary(RT_SOFTPLUS, x); }
  static Storage square(const Storage& x) { return unary(RT_SQUARE, x); }
  static Storage elu(const Storage& x, float alpha) { return unary(RT_ELU, x, alpha); }
  static Storage clip(const Storage& x, float lo, float hi) { return unary(RT_CLIP, x, lo, hi); }
  static Storage sqrt(const Storage& x) {
    // The reference rejects any negative input (src/backend/cpu.rs:1717-1723); the check
    // is a device min-reduction read back to the host.
    if (x.numel() > 0) {
      Storage m = min(x, std::nullopt);
      if (copy_to_host(m).at(0) < 0.0f) throw Error::invalid_op("sqrt: input contains negative values");
    }
    return unary(RT_SQRT, x);
  }
  static Storage relu_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_RELU, o, g); }
  static Storage elu_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_ELU, o, g, o.op_type.scalar); }
  static Storage exp_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_EXP, o, g); }
  static Storage ln_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_LN, o, g); }
  static Storage abs_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_ABS, o, g); }
  static Storage sigmoid_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_SIGMOID, o, g); }
  static Storage tanh_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_TANH, o, g); }
  static Storage sqrt_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_SQRT, o, g); }
  static Storage softplus_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_SOFTPLUS, o, g); }
  static Storage square_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_SQUARE, o, g); }
  static Storage sin_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_SIN, o, g); }
  static Storage cos_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_COS, o, g); }
  static Storage tan_backward(const OpB& o, const Storage& g) { return unary_bwd(RT_TAN, o, g); }
  static Storage clip_backward(const OpB& o, const Storage& g) {
    return unary_bwd(RT_CLIP, o, g, o.op_type.min_val, o.op_type.max_val);
  }

  // ---- layout -----------------------------------------------------------------------------
  static Storage transpose(const Storage& x) {
    if (x.shape.size() <= 1) return x;
    if (x.shape.size() != 2) throw Error::unimplemented("transpose of more than 2 dimensions");
    Storage y = alloc(Shape{x.shape[1], x.shape[0]});
    check(rt_transpose2d(ctx(), x.ptr(), (int64_t)x.shape[0], (int64_t)x.shape[1], y.ptr()));
    return y;
  }
  static Storage broadcast_to(const Storage& x, const Shape& shape) {
    if (shape.size() < x.shape.size()) throw Error::incompatible("broadcast", x.shape, shape);
    size_t off = shape.size() - x.shape.size();
    for (size_t i = 0; i < x.shape.size(); ++i)
      if (x.shape[i] != shape[i + off] && x.shape[i] != 1) throw Error::incompatible("broadcast", x.shape, shape);
    Storage y = alloc(shape);
    auto xs = dims(x.shape), os = dims(shape);
    check(rt_broadcast_to(ctx(), x.ptr(), xs.data(), (int)xs.size(), os.data(), (int)os.size(), y.ptr()));
    return y;
  }
  static Storage unbroadcast(const Storage& g, const Shape& target) {
    if (g.shape == target) return g;
    // The reduction works on the right-aligned target; a target that is rank-compatible
    // only after reshaping (same element count) is reshaped, as the reference does last.
    Shape t = target;
    auto gs = dims(g.shape), ts = dims(t);
    if (ts.size() > gs.size()) {
      if (shape_numel(t) == g.numel()) {
        Storage r = g;
        r.shape = t;
        return r;
      }
      throw Error::incompatible("unbroadcast (final shape/size)", g.shape, target);
    }
    Storage out = alloc(t);
    check(rt_unbroadcast(ctx(), g.ptr(), gs.data(), (int)gs.size(), ts.data(), (int)ts.size(), out.ptr()));
    return out;
  }
  static Storage slice(const Storage& x, const std::vector<Range>& ranges) {
    if (ranges.size() != x.shape.size()) throw Error::invalid_op("Slice ranges do not match input dimensionality");
    Shape os(ranges.size());
    std::vector<int64_t> starts(ranges.size());
    for (size_t i = 0; i < ranges.size(); ++i) {
      os[i] = ranges[i].end - ranges[i].start;
      starts[i] = (int64_t)ranges[i].start;
    }
    Storage y = alloc(os);
    auto xs = dims(x.shape), od = dims(os);
    check(rt_slice(ctx(), x.ptr(), xs.data(), (int)xs.size(), starts.data(), od.data(), y.ptr()));
    return y;
  }
  static Storage slice_backward(const OpB& o, const Storage& g) {
    if (o.op_type.kind != OpType::Slice) throw Error::internal("Incorrect OpType for slice_backward");
    const Shape& is = o.op_type.input_shape;
    std::vector<int64_t> starts;
    Shape gs;
    for (auto& r : o.op_type.ranges) {
      starts.push_back((int64_t)r.start);
      gs.push_back(r.end - r.start);
    }
    if (shape_numel(gs) != g.numel()) throw Error::incompatible("slice_backward", gs, g.shape);
    Storage dx = zeros(is);
    auto id = dims(is), gd = dims(gs);
    check(rt_slice_assign(ctx(), dx.ptr(), id.data(), (int)id.size(), starts.data(), g.ptr(), gd.data()));
    return dx;
  }
  static Storage concat(const std::vector<const Storage*>& xs, size_t axis) {
    if (xs.empty()) throw Error::invalid_op("Cannot concat empty list of storages");
    Shape os = xs[0]->shape;
    if (axis >= os.size()) throw Error(ErrorKind::ShapeError, "concatenate: axis out of bounds");
    size_t total = 0;
    for (auto* x : xs) {
      if (x->shape.size() != os.size()) throw Error(ErrorKind::ShapeError, "concatenate: incompatible shapes");
      for (size_t d = 0; d < os.size(); ++d)
        if (d != axis && x->shape[d] != os[d]) throw Error(ErrorKind::ShapeError, "concatenate: incompatible shapes");
      total += x->shape[axis];
    }
    os[axis] = total;
    Storage y = alloc(os);
    auto od = dims(os);
    std::vector<int64_t> starts(os.size(), 0);
    for (auto* x : xs) {
      auto xd = dims(x->shape);
      check(rt_slice_assign(ctx(), y.ptr(), od.data(), (int)od.size(), starts.data(), x->ptr(), xd.data()));
      starts[axis] += (int64_t)x->shape[axis];
    }
    return y;
  }
  // concat({x[r0:r1, :], h}, axis 1) for 2-D x and h without materialising the row slice: rows r0..r1 of a row-major matrix are
  // one contiguous block, which goes straight into the left columns of the result.
  static Storage concat_rows_with(const Storage& x, size_t r0, size_t r1, const Storage& h) {
    if (x.shape.size() != 2 || h.shape.size() != 2 || r0 > r1 || r1 > x.shape[0] || h.shape[0] != r1 - r0)
      throw Error(ErrorKind::ShapeError, "concat_rows_with: incompatible shapes");
    Shape os{r1 - r0, x.shape[1] + h.shape[1]};
    Storage y = alloc(os);
    auto od = dims(os);
    std::vector<int64_t> starts{0, 0};
    Shape xs{r1 - r0, x.shape[1]};
    auto xd = dims(xs), hd = dims(h.shape);
    if (shape_numel(xs) > 0) check(rt_slice_assign(ctx(), y.ptr(), od.data(), 2, starts.data(), x.ptr() + r0 * x.shape[1], xd.data()));
    starts[1] = (int64_t)x.shape[1];
    if (h.numel() > 0) check(rt_slice_assign(ctx(), y.ptr(), od.data(), 2, starts.data(), h.ptr(), hd.data()));
    return y;
  }
  static std::vector<Storage> concat_backward(const OpB& o, const Storage& g) {
    if (o.op_type.kind != OpType::Concat) throw Error::internal("Incorrect OpType for concat_backward");
    size_t axis = *o.op_type.axis;
    std::vector<Storage> grads;
    size_t off = 0;
    for (size_t i = 0; i < o.op_type.input_shapes.size(); ++i) {
      const Shape& s = o.op_type.input_shapes[i];
      if (i < o.inputs.size() && !o.inputs[i].requires_grad()) {
        grads.push_back(Storage{nullptr, s});  // never accumulated
      } else {
        std::vector<Range> r;
        for (size_t d = 0; d < g.shape.size(); ++d) r.push_back(d == axis ? Range{off, off + s[axis]} : Range{0, g.shape[d]});
        grads.push_back(slice(g, r));
      }
      off += s[axis];
    }
    return grads;
  }
  static Storage expand_dims(const Storage& x, size_t axis) {
    if (axis > x.shape.size()) throw Error::invalid_index(axis);
    Storage y = x;
    y.shape.insert(y.shape.begin() + axis, 1);
    return y;
  }
  static Storage expand_dims_backward(const OpB& o, const Storage& g) {
    size_t axis = *o.op_type.axis;
    Shape orig = o.inputs[0].shape();
    Storage out = g;
    if (axis < g.shape.size() && g.shape[axis] == 1) {
      set_shape(out, orig);
    } else if (axis < g.shape.size()) {
      out = sum_along_axis(g, axis);
      set_shape(out, orig);
    } else {
      throw Error::internal("expand_dims_backward: axis out of bounds for grad_output");
    }
    return out;
  }
  static Storage squeeze(const Storage& x, std::optional<size_t> axis) {
    Shape ns;
    if (axis) {
      if (*axis >= x.shape.size()) throw Error::invalid_index(*axis);
      if (x.shape[*axis] != 1) throw Error::invalid_op("Cannot squeeze axis (not size 1)");
      ns = x.shape;
      ns.erase(ns.begin() + *axis);
    } else {
      for (size_t d : x.shape)
        if (d != 1) ns.push_back(d);
    }
    Storage y = x;
    set_shape(y, ns);
    return y;
  }
  static Storage squeeze_backward(const OpB& o, const Storage& g) {
    Storage y = g;
    set_shape(y, o.op_type.input_shape);
    return y;
  }

  // ---- reductions ---------------------------------------------------------------------------
  struct Axis3 {
    int64_t outer, len, inner;
    Shape out_shape;
  };
  static Axis3 split(const Shape& s, std::optional<size_t> axis) {
    Axis3 a{1, 1, 1, {}};
    if (!axis) {
      a.len = (int64_t)shape_numel(s);
      return a;
    }
    if (*axis >= s.size()) throw Error::invalid_index(*axis);
    for (size_t d = 0; d < *axis; ++d) a.outer *= (int64_t)s[d];
    a.len = (int64_t)s[*axis];
    for (size_t d = *axis + 1; d < s.size(); ++d) a.inner *= (int64_t)s[d];
    a.out_shape = s;
    a.out_shape.erase(a.out_shape.begin() + *axis);
    return a;
  }
  static Storage reduce(int kind, const Storage& x, std::optional<size_t> axis) {
    Axis3 a = split(x.shape, axis);
    Storage out = alloc(a.out_shape);
    check(rt_reduce(ctx(), kind, x.ptr(), a.outer, a.len, a.inner, out.ptr()));
    return out;
  }
  static Storage sum_along_axis(const Storage& x, size_t axis) { return reduce(RT_RED_SUM, x, axis); }
  static Storage max_along_axis(const Storage& x, size_t axis) { return reduce(RT_RED_MAX, x, axis); }
  static float sum_all(const Storage& x) {
    float v = 0.f;
    check(rt_sum_all_host(ctx(), x.ptr(), (int64_t)x.numel(), &v));
    return v;
  }
  static Storage sum_all_scalar(const Storage& x) { return reduce(RT_RED_SUM, x, std::nullopt); }
  static Storage mean(const Storage& x, std::optional<size_t> axis) {
    if (axis) {
      if (*axis >= x.shape.size()) throw Error::invalid_index(*axis);
      if (x.shape[*axis] == 0) throw Error::invalid_op("Mean failed along axis");
    } else if (x.numel() == 0) {
      throw Error(ErrorKind::EmptyTensor, "empty tensor");
    }
    return reduce(RT_RED_MEAN, x, axis);
  }
  static Storage reduce_or_empty(int kind, const Storage& x, std::optional<size_t> axis) {
    if (x.numel() == 0) return zeros(x.shape);
    return reduce(kind, x, axis);
  }
  static Storage max(const Storage& x, std::optional<size_t> axis) { return reduce_or_empty(RT_RED_MAX, x, axis); }
  static Storage min(const Storage& x, std::optional<size_t> axis) { return reduce_or_empty(RT_RED_MIN, x, axis); }
  static Storage prod(const Storage& x, std::optional<size_t> axis) { return reduce_or_empty(RT_RED_PROD, x, axis); }
  static Storage logsumexp(const Storage& x, std::optional<size_t> axis) { return reduce_or_empty(RT_RED_LOGSUMEXP, x, axis); }
  static Storage argmax(const Storage& x, size_t axis) { return reduce_or_empty(RT_RED_ARGMAX, x, axis); }
  static Storage argmin(const Storage& x, size_t axis) { return reduce_or_empty(RT_RED_ARGMIN, x, axis); }
  static Storage log_softmax(const Storage& x, size_t axis) {
    Axis3 a = split(x.shape, axis);
    Storage y = alloc(x.shape);
    check(rt_log_softmax(ctx(), x.ptr(), a.outer, a.len, a.inner, y.ptr()));
    return y;
  }
  static Storage reduce_bwd(int kind, const OpB& o, const Storage& g, const char* name) {
    if (o.inputs.size() != 1) throw Error::invalid_op(std::string(name) + " backward expects 1 input");
    const Storage& x = o.inputs[0].data();
    Axis3 a = split(x.shape, o.op_type.axis);
    if ((int64_t)g.numel() != a.outer * a.inner) throw Error::incompatible(name, x.shape, g.shape);
    Storage dx = alloc(x.shape);
    check(rt_reduce_backward(ctx(), kind, x.ptr(), g.ptr(), a.outer, a.len, a.inner, dx.ptr()));
    return dx;
  }
  static Storage sum_backward(const OpB& o, const Storage& g) {
    if (!o.op_type.axis && !g.shape.empty()) throw Error::shape_mismatch(Shape{}, g.shape);  // cpu.rs:1480-1485
    return reduce_bwd(RT_RED_SUM, o, g, "sum");
  }
  static Storage mean_backward(const OpB& o, const Storage& g) { return reduce_bwd(RT_RED_MEAN, o, g, "mean"); }
  static Storage max_backward(const OpB& o, const Storage& g) { return reduce_bwd(RT_RED_MAX, o, g, "max"); }
  static Storage min_backward(const OpB& o, const Storage& g) { return reduce_bwd(RT_RED_MIN, o, g, "min"); }
  static Storage prod_backward(const OpB& o, const Storage& g) { return reduce_bwd(RT_RED_PROD, o, g, "prod"); }
  static Storage logsumexp_backward(const OpB& o, const Storage& g) { return reduce_bwd(RT_RED_LOGSUMEXP, o, g, "logsumexp"); }
  static Storage log_softmax_backward(const OpB& o, const Storage& g) {
    if (o.inputs.empty()) throw Error::invalid_op("LogSoftmax requires 1 input");
    const Storage& x = o.inputs[0].data();
    Axis3 a = split(x.shape, o.op_type.axis);
    if (g.shape != x.shape) throw Error::shape_mismatch(x.shape, g.shape);
    Storage dx = alloc(x.shape);
    check(rt_log_softmax_backward(ctx(), x.ptr(), g.ptr(), a.outer, a.len, a.inner, dx.ptr()));
    return dx;
  }

  // ---- contractions / pooling -------------------------------------------------------------------
  static Storage matmul(const Storage& a, const Storage& b) {
    if (a.shape.size() != 2) throw Error(ErrorKind::ShapeError, "Input 'a' is not 2D");
    if (b.shape.size() != 2) throw Error(ErrorKind::ShapeError, "Input 'b' is not 2D");
    if (a.shape[1] != b.shape[0]) throw Error::incompatible("matmul", a.shape, b.shape);
    int64_t m = (int64_t)a.shape[0], k = (int64_t)a.shape[1], n = (int64_t)b.shape[1];
    Storage c = alloc(Shape{a.shape[0], b.shape[1]});
    check(rt_gemm(ctx(), 0, 0, m, n, k, a.ptr(), k, b.ptr(), n, c.ptr(), n, 0));
    return c;
  }
  static std::pair<Storage, Storage> matmul_backward(const OpB& o, const Storage& g) {
    if (o.inputs.size() != 2) throw Error::invalid_op("Matmul requires 2 inputs");
    const Storage& a = o.inputs[0].data();
    const Storage& b = o.inputs[1].data();
    int64_t m = (int64_t)a.shape[0], k = (int64_t)a.shape[1], n = (int64_t)b.shape[1];
    if (g.shape != Shape{a.shape[0], b.shape[1]}) throw Error::incompatible("matmul", g.shape, b.shape);
    bool need_a = o.inputs[0].requires_grad(), need_b = o.inputs[1].requires_grad();
    Storage da = need_a ? alloc(a.shape) : Storage{nullptr, a.shape};
    Storage db = need_b ? alloc(b.shape) : Storage{nullptr, b.shape};
    check(rt_matmul_backward(ctx(), a.ptr(), b.ptr(), g.ptr(), m, k, n, da.ptr(), db.ptr()));
    return {std::move(da), std::move(db)};
  }
  static std::pair<Storage, Storage> matmul_closure_backward(const OpB& o, const Storage& g) { return matmul_backward(o, g); }
  // matmul backward when the second operand already holds a gradient: returns dA and adds A^T g to `acc` in place (the
  // product kernel accumulates into its output; one launch instead of a product and an addition)
  static Storage matmul_backward_accumulate(const OpB& o, const Storage& g, Storage& acc) {
    const Storage& a = o.inputs[0].data();
    const Storage& b = o.inputs[1].data();
    int64_t m = (int64_t)a.shape[0], k = (int64_t)a.shape[1], n = (int64_t)b.shape[1];
    if (g.shape != Shape{a.shape[0], b.shape[1]}) throw Error::incompatible("matmul", g.shape, b.shape);
    if (acc.shape != b.shape) throw Error::shape_mismatch(b.shape, acc.shape);
    Storage da = o.inputs[0].requires_grad() ? alloc(a.shape) : Storage{nullptr, a.shape};
    make_unique(acc);  // nobody else may see the sum appear in a buffer they share
    check(rt_matmul_backward_accumulate(ctx(), a.ptr(), b.ptr(), g.ptr(), m, k, n, da.ptr(), acc.ptr()));
    return da;
  }
  static bool is_accumulated(const Storage& s) { return !s.buf; }
  // the accumulating epilogue of the product works on 128-bit pieces of a row; other widths keep product + addition
  static bool accumulates_well(const Storage& b) { return b.shape.size() == 2 && b.shape[1] % 4 == 0; }

  static void conv_shapes(const Storage& x, const Storage& w, const char* name) {
    if (x.shape.size() != 4 || w.shape.size() != 4) throw Error::invalid_op(std::string(name) + " expects 4D input and weights");
  }
  static Storage conv2d(const Storage& x, const Storage& w, const Storage* bias, Pair s, Pair p) {
    conv_shapes(x, w, "conv2d");
    if (x.shape[1] != w.shape[1]) throw Error::invalid_op("conv2d: input channels != weight channels");
    if (bias && bias->numel() != w.shape[0]) throw Error::invalid_op("conv2d: bias shape mismatch");
    size_t ho = (x.shape[2] + 2 * p.first - w.shape[2]) / s.first + 1, wo = (x.shape[3] + 2 * p.second - w.shape[3]) / s.second + 1;
    Storage y = alloc(Shape{x.shape[0], w.shape[0], ho, wo});
    check(rt_conv2d(ctx(), x.ptr(), w.ptr(), bias ? bias->ptr() : nullptr, (int64_t)x.shape[0], (int64_t)x.shape[1],
                    (int64_t)x.shape[2], (int64_t)x.shape[3], (int64_t)w.shape[0], (int)w.shape[2], (int)w.shape[3],
                    (int)s.first, (int)s.second, (int)p.first, (int)p.second, y.ptr()));
    return y;
  }
  static std::tuple<Storage, Storage, std::optional<Storage>> conv2d_backward(const Storage& x, const Storage& w,
                                                                              const Storage& g, Pair s, Pair p,
                                                                              bool need_x = true, bool need_w = true,
                                                                              bool need_b = true) {
    conv_shapes(x, w, "conv2d_backward");
    size_t ho = (x.shape[2] + 2 * p.first - w.shape[2]) / s.first + 1, wo = (x.shape[3] + 2 * p.second - w.shape[3]) / s.second + 1;
    Shape gs{x.shape[0], w.shape[0], ho, wo};
    if (g.shape != gs) throw Error::shape_mismatch(gs, g.shape);
    Storage dx = need_x ? alloc(x.shape) : Storage{nullptr, x.shape};
    Storage dw = need_w ? alloc(w.shape) : Storage{nullptr, w.shape};
    Storage db = need_b ? alloc(Shape{w.shape[0]}) : Storage{nullptr, Shape{w.shape[0]}};
    check(rt_conv2d_backward(ctx(), x.ptr(), w.ptr(), g.ptr(), (int64_t)x.shape[0], (int64_t)x.shape[1], (int64_t)x.shape[2],
                             (int64_t)x.shape[3], (int64_t)w.shape[0], (int)w.shape[2], (int)w.shape[3], (int)s.first,
                             (int)s.second, (int)p.first, (int)p.second, dx.ptr(), dw.ptr(), db.ptr()));
    return {std::move(dx), std::move(dw), std::optional<Storage>(std::move(db))};
  }
  // max_pool2d(relu(conv2d(x, w) + bias), 2x2, stride 2) without keeping the convolution output: {pooled values, indices}
  static std::pair<Storage, Storage> conv2d_relu_max_pool2x2(const Storage& x, const Storage& w, const Storage* bias, Pair s, Pair p) {
    conv_shapes(x, w, "conv2d_relu_max_pool2x2");
    if (x.shape[1] != w.shape[1]) throw Error::invalid_op("conv2d_relu_max_pool2x2: input channels != weight channels");
    if (bias && bias->numel() != w.shape[0]) throw Error::invalid_op("conv2d_relu_max_pool2x2: bias shape mismatch");
    size_t ho = (x.shape[2] + 2 * p.first - w.shape[2]) / s.first + 1, wo = (x.shape[3] + 2 * p.second - w.shape[3]) / s.second + 1;
    if ((ho & 1) || (wo & 1)) throw Error::invalid_op("conv2d_relu_max_pool2x2: the convolution output must have even extents");
    Storage y = alloc(Shape{x.shape[0], w.shape[0], ho / 2, wo / 2}), idx = alloc(Shape{x.shape[0], w.shape[0], ho / 2, wo / 2});
    check(rt_conv2d_relu_max_pool2x2(ctx(), x.ptr(), w.ptr(), bias ? bias->ptr() : nullptr, (int64_t)x.shape[0], (int64_t)x.shape[1],
                                     (int64_t)x.shape[2], (int64_t)x.shape[3], (int64_t)w.shape[0], (int)w.shape[2], (int)w.shape[3],
                                     (int)s.first, (int)s.second, (int)p.first, (int)p.second, y.ptr(), idx.ptr()));
    return {std::move(y), std::move(idx)};
  }
  // Its backward: the gradient of the convolution output from the pooled output and the indices, then conv2d_backward.
  static std::tuple<Storage, Storage, std::optional<Storage>> conv2d_relu_max_pool2x2_backward(
      const Storage& x, const Storage& w, const Storage& y, const Storage& idx, const Storage& g, Pair s, Pair p, bool need_x, bool need_w,
      bool need_b) {
    if (g.shape != y.shape) throw Error::shape_mismatch(y.shape, g.shape);
    Storage dconv = alloc(Shape{y.shape[0], y.shape[1], y.shape[2] * 2, y.shape[3] * 2});
    check(rt_relu_max_pool2x2_backward_from_output(ctx(), y.ptr(), g.ptr(), idx.ptr(), (int64_t)y.shape[0], (int64_t)y.shape[1],
                                                   (int64_t)y.shape[2] * 2, (int64_t)y.shape[3] * 2, dconv.ptr()));
    return conv2d_backward(x, w, dconv, s, p, need_x, need_w, need_b);
  }
  static Storage conv2d_transpose(const Storage& x, const Storage& w, const Storage* bias, Pair s, Pair p) {
    if (x.shape.size() != 4) throw Error(ErrorKind::ShapeError, "Expected 4D input tensor for conv2d_transpose");
    if (w.shape.size() != 4) throw Error(ErrorKind::ShapeError, "Expected 4D weights tensor for conv2d_transpose");
    if (x.shape[1] != w.shape[0]) throw Error::shape_mismatch(Shape{x.shape[0], w.shape[0], x.shape[2], x.shape[3]}, x.shape);
    if (bias && (bias->shape.size() != 1 || bias->shape[0] != w.shape[1])) throw Error::shape_mismatch(Shape{w.shape[1]}, bias->shape);
    size_t oh = (x.shape[2] - 1) * s.first + w.shape[2] - 2 * p.first, ow = (x.shape[3] - 1) * s.second + w.shape[3] - 2 * p.second;
    Storage y = alloc(Shape{x.shape[0], w.shape[1], oh, ow});
    check(rt_conv2d_transpose(ctx(), x.ptr(), w.ptr(), bias ? bias->ptr() : nullptr, (int64_t)x.shape[0], (int64_t)x.shape[1],
                              (int64_t)x.shape[2], (int64_t)x.shape[3], (int64_t)w.shape[1], (int)w.shape[2], (int)w.shape[3],
                              (int)s.first, (int)s.second, (int)p.first, (int)p.second, y.ptr()));
    return y;
  }
  static std::tuple<Storage, Storage, std::optional<Storage>> conv2d_transpose_backward(const Storage& x, const Storage& w,
                                                                                        const Storage& g, Pair s, Pair p,
                                                                                        bool need_x = true, bool need_w = true,
                                                                                        bool need_b = true) {
    if (x.shape.size() != 4 || w.shape.size() != 4 || g.shape.size() != 4)
      throw Error(ErrorKind::ShapeError, "Expected 4D tensors for conv2d_transpose_backward");
    if (x.shape[1] != w.shape[0]) throw Error::shape_mismatch(Shape{x.shape[0], w.shape[0], x.shape[2], x.shape[3]}, x.shape);
    if (g.shape[1] != w.shape[1]) throw Error::shape_mismatch(Shape{x.shape[0], w.shape[1], g.shape[2], g.shape[3]}, g.shape);
    size_t oh = (x.shape[2] - 1) * s.first + w.shape[2] - 2 * p.first, ow = (x.shape[3] - 1) * s.second + w.shape[3] - 2 * p.second;
    if (g.shape[2] != oh || g.shape[3] != ow || g.shape[0] != x.shape[0])
      throw Error::shape_mismatch(Shape{x.shape[0], w.shape[1], oh, ow}, g.shape);
    Storage dx = need_x ? alloc(x.shape) : Storage{nullptr, x.shape};
    Storage dw = need_w ? alloc(w.shape) : Storage{nullptr, w.shape};
    Storage db = need_b ? alloc(Shape{w.shape[1]}) : Storage{nullptr, Shape{w.shape[1]}};
    check(rt_conv2d_transpose_backward(ctx(), x.ptr(), w.ptr(), g.ptr(), (int64_t)x.shape[0], (int64_t)x.shape[1],
                                       (int64_t)x.shape[2], (int64_t)x.shape[3], (int64_t)w.shape[1], (int)w.shape[2],
                                       (int)w.shape[3], (int)s.first, (int)s.second, (int)p.first, (int)p.second, dx.ptr(),
                                       dw.ptr(), db.ptr()));
    return {std::move(dx), std::move(dw), std::optional<Storage>(std::move(db))};
  }
  static std::pair<Storage, Storage> max_pool2d(const Storage& x, Pair k, Pair s, Pair p) {
    if (x.shape.size() != 4) throw Error::invalid_op("max_pool2d expects 4D input (NCHW)");
    size_t ho = (x.shape[2] + 2 * p.first - k.first) / s.first + 1, wo = (x.shape[3] + 2 * p.second - k.second) / s.second + 1;
    Shape os{x.shape[0], x.shape[1], ho, wo};
    Storage y = alloc(os), idx = alloc(os);
    check(rt_max_pool2d(ctx(), x.ptr(), (int64_t)x.shape[0], (int64_t)x.shape[1], (int64_t)x.shape[2], (int64_t)x.shape[3],
                        (int)k.first, (int)k.second, (int)s.first, (int)s.second, (int)p.first, (int)p.second, y.ptr(),
                        idx.ptr()));
    return {std::move(y), std::move(idx)};
  }
  static Storage max_pool2d_backward(const OpB& o, const Storage& g) {
    if (o.inputs.size() < 2) throw Error::invalid_op("max_pool2d_backward requires at least 2 inputs (input and indices)");
    if (o.op_type.kind != OpType::MaxPool2D) throw Error::internal("Expected MaxPool2d op type for max_pool2d_backward");
    Shape is = o.inputs[0].shape();
    const Storage& idx = o.inputs[1].data();
    if (g.numel() != idx.numel()) throw Error::shape_mismatch(idx.shape, g.shape);
    Pair k = o.op_type.kernel_size, s = o.op_type.stride, p = o.op_type.padding;
    Storage dx = alloc(is);
    check(rt_max_pool2d_backward(ctx(), g.ptr(), idx.ptr(), (int64_t)is[0], (int64_t)is[1], (int64_t)is[2], (int64_t)is[3],
                                 (int)k.first, (int)k.second, (int)s.first, (int)s.second, (int)p.first, (int)p.second,
                                 dx.ptr()));
    return dx;
  }

  // ---- fused forward ops (no counterpart in the reference; ops::fused_* in autograd.hpp) -------------------------
  static std::pair<Storage, Storage> relu_max_pool2d(const Storage& x, Pair k, Pair s, Pair p) {
    if (x.shape.size() != 4) throw Error::invalid_op("relu_max_pool2d expects 4D input (NCHW)");
    size_t ho = (x.shape[2] + 2 * p.first - k.first) / s.first + 1, wo = (x.shape[3] + 2 * p.second - k.second) / s.second + 1;
    Shape os{x.shape[0], x.shape[1], ho, wo};
    Storage y = alloc(os), idx = alloc(os);
    check(rt_relu_max_pool2d(ctx(), x.ptr(), (int64_t)x.shape[0], (int64_t)x.shape[1], (int64_t)x.shape[2], (int64_t)x.shape[3],
                             (int)k.first, (int)k.second, (int)s.first, (int)s.second, (int)p.first, (int)p.second, y.ptr(),
                             idx.ptr()));
    return {std::move(y), std::move(idx)};
  }
  static Storage relu_max_pool2d_backward(const OpB& o, const Storage& g) {
    if (o.inputs.size() < 2) throw Error::invalid_op("relu_max_pool2d_backward requires the input and the indices");
    const Storage& x = o.inputs[0].data();
    const Storage& idx = o.inputs[1].data();
    if (g.numel() != idx.numel()) throw Error::shape_mismatch(idx.shape, g.shape);
    Shape is = x.shape;
    Pair k = o.op_type.kernel_size, s = o.op_type.stride, p = o.op_type.padding;
    Storage dx = alloc(is);
    check(rt_relu_max_pool2d_backward(ctx(), x.ptr(), g.ptr(), idx.ptr(), (int64_t)is[0], (int64_t)is[1], (int64_t)is[2],
                                      (int64_t)is[3], (int)k.first, (int)k.second, (int)s.first, (int)s.second, (int)p.first,
                                      (int)p.second, dx.ptr()));
    return dx;
  }
  static Storage softmax_nll(const Storage& logits, const Storage& targets) {
    Storage loss = alloc(Shape{});
    check(rt_softmax_cross_entropy(ctx(), logits.ptr(), targets.ptr(), (int64_t)logits.shape[0], (int64_t)logits.shape[1],
                                   loss.ptr()));
    return loss;
  }
  static std::pair<Storage, Storage> softmax_nll_backward(const OpB& o, const Storage& g) {
    const Storage& logits = o.inputs[0].data();
    const Storage& targets = o.inputs[1].data();
    if (g.numel() != 1) throw Error::shape_mismatch(Shape{}, g.shape);
    const bool need_l = o.inputs[0].requires_grad(), need_t = o.inputs[1].requires_grad();
    Storage dl = need_l ? alloc(logits.shape) : unused_grad(logits.shape);
    Storage dt = need_t ? alloc(targets.shape) : unused_grad(targets.shape);
    check(rt_softmax_cross_entropy_backward(ctx(), logits.ptr(), targets.ptr(), g.ptr(), (int64_t)logits.shape[0],
                                            (int64_t)logits.shape[1], need_l ? dl.ptr() : nullptr, need_t ? dt.ptr() : nullptr));
    return {std::move(dl), std::move(dt)};
  }

  static Storage lstm_cell_c(const Storage& gates, const Storage& c_prev) {
    Storage c = alloc(c_prev.shape);
    check(rt_lstm_cell_c(ctx(), gates.ptr(), c_prev.ptr(), (int64_t)c_prev.shape[0], (int64_t)c_prev.shape[1], c.ptr()));
    return c;
  }
  static std::pair<Storage, Storage> lstm_cell_c_backward(const OpB& o, const Storage& g) {
    const Storage& gates = o.inputs[0].data();
    const Storage& c_prev = o.inputs[1].data();
    if (g.shape != c_prev.shape) throw Error::shape_mismatch(c_prev.shape, g.shape);
    const bool ng = o.inputs[0].requires_grad(), nc = o.inputs[1].requires_grad();
    Storage dg = ng ? alloc(gates.shape) : unused_grad(gates.shape);
    Storage dc = nc ? alloc(c_prev.shape) : unused_grad(c_prev.shape);
    check(rt_lstm_cell_c_backward(ctx(), gates.ptr(), c_prev.ptr(), g.ptr(), (int64_t)c_prev.shape[0], (int64_t)c_prev.shape[1],
                                  ng ? dg.ptr() : nullptr, nc ? dc.ptr() : nullptr));
    return {std::move(dg), std::move(dc)};
  }
  static Storage lstm_cell_h(const Storage& gates, const Storage& c) {
    Storage h = alloc(c.shape);
    check(rt_lstm_cell_h(ctx(), gates.ptr(), c.ptr(), (int64_t)c.shape[0], (int64_t)c.shape[1], h.ptr()));
    return h;
  }
  static std::pair<Storage, Storage> lstm_cell_h_backward(const OpB& o, const Storage& g) {
    const Storage& gates = o.inputs[0].data();
    const Storage& c = o.inputs[1].data();
    if (g.shape != c.shape) throw Error::shape_mismatch(c.shape, g.shape);
    const bool ng = o.inputs[0].requires_grad(), nc = o.inputs[1].requires_grad();
    Storage dg = ng ? alloc(gates.shape) : unused_grad(gates.shape);
    Storage dc = nc ? alloc(c.shape) : unused_grad(c.shape);
    check(rt_lstm_cell_h_backward(ctx(), gates.ptr(), c.ptr(), g.ptr(), (int64_t)c.shape[0], (int64_t)c.shape[1],
                                  ng ? dg.ptr() : nullptr, nc ? dc.ptr() : nullptr));
    return {std::move(dg), std::move(dc)};
  }

  // ---- optimizer steps (mod.rs:18-36, 256-272) ---------------------------------------------------
  static void sgd_step(Storage& w, const Storage& dw, float lr) {
    if (w.shape != dw.shape) throw Error::shape_mismatch(w.shape, dw.shape);
    make_unique(w);
    check(rt_sgd_step(ctx(), w.ptr(), dw.ptr(), (int64_t)w.numel(), lr));
  }
  static void momentum_sgd_step(Storage& p, const Storage& g, Storage& vel, float lr, float mu) {
    if (p.shape != vel.shape) throw Error::shape_mismatch(p.shape, vel.shape);
    if (p.shape != g.shape) throw Error::shape_mismatch(p.shape, g.shape);
    make_unique(p);
    make_unique(vel);
    check(rt_momentum_sgd_step(ctx(), p.ptr(), g.ptr(), vel.ptr(), (int64_t)p.numel(), lr, mu));
  }
  static void adagrad_step(Storage& p, const Storage& g, Storage& acc, float lr, float eps) {
    if (p.shape != g.shape) throw Error::shape_mismatch(p.shape, g.shape);
    if (p.shape != acc.shape) throw Error::shape_mismatch(p.shape, acc.shape);
    make_unique(p);
    make_unique(acc);
    check(rt_adagrad_step(ctx(), p.ptr(), g.ptr(), acc.ptr(), (int64_t)p.numel(), lr, eps));
  }
  static void adam_step(Storage& p, const Storage& g, Storage& m, Storage& v, float lr, float b1, float b2, float eps,
                        size_t t) {
    if (p.shape != g.shape) throw Error::shape_mismatch(p.shape, g.shape);
    if (p.shape != m.shape) throw Error::shape_mismatch(p.shape, m.shape);
    if (p.shape != v.shape) throw Error::shape_mismatch(p.shape, v.shape);
    if (t == 0) throw Error::internal("Adam step called with t=0");
    make_unique(p);
    make_unique(m);
    make_unique(v);
    check(rt_adam_step(ctx(), p.ptr(), g.ptr(), m.ptr(), v.ptr(), (int64_t)p.numel(), lr, b1, b2, eps, (int64_t)t));
  }
};

}  // namespace rt
