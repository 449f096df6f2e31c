// ORACLE -- test infrastructure, not product code.
//
// A single-threaded C++ restatement of the reference library's CPU backend
// (`CpuBackend` on ndarray), used only as the checker for the CUDA path and as
// the timed CPU baseline.  Nothing in the shipped library may include, link or
// call this file.
//
// Parity status: pinned against the known-answer tests of the reference
// (tests/ops_cpu_tests.rs, tests/ops_cpu_backward_tests.rs, tests/optim_tests.rs,
// tests/test_concat.rs, src/optim.rs inline tests) for elementwise ops,
// reductions, broadcasting, accumulation, slice/concat/clip and the optimizers.
// PARITY UNPINNED for conv2d / conv2d_backward / conv2d_transpose(_backward) and
// max_pool2d_backward: the reference has no CPU test for them, so this file's
// restatement of the reference source is the only specification; those functions
// are additionally cross-checked against float64 direct convolutions and finite
// differences in tests/.
//
// The arithmetic that the reference delegates to third-party crates that are
// not part of its source tree is restated from their published algorithms:
//   ndarray 0.16.1        sum_axis / sum (eight-way unrolled fold), fold_axis, mean_axis, broadcast
//   matrixmultiply 0.3.9  sgemm (fp32 accumulation; only the summation order differs here)
//   compiler-rt           __powisf2 for f32::powi (repeated squaring)
//
// Every function cites the reference file:line it follows.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <optional>
#include <tuple>
#include <random>
#include <vector>

#include "../rusttensor_b200/csrc/host/autograd.hpp"

namespace oracle {

using rt::Error;
using rt::ErrorKind;
using rt::Op;
using rt::OpType;
using rt::Pair;
using rt::Range;
using rt::Shape;
using rt::shape_numel;

// When true (default) conv2d_backward reproduces the reference's input-gradient
// defect (src/ops/cpu_ops.rs:266,271: `col_idx` is never advanced, so every
// output pixel scatters column 0).  When false the column index follows the
// output pixel, which is the mathematically correct col2im.
inline bool& conv_dx_faithful() {
  static bool v = true;
  return v;
}

// src/array.rs:14-18 -- owned, C-contiguous f32 array with a dynamic shape.
struct Array {
  std::vector<float> data;
  Shape shape;
  Array() = default;
  Array(std::vector<float> d, Shape s) : data(std::move(d)), shape(std::move(s)) {}
  static Array filled(const Shape& s, float v) { return Array(std::vector<float>(shape_numel(s), v), s); }
  size_t size() const { return data.size(); }
  size_t ndim() const { return shape.size(); }
};

// ---- ndarray numeric_util::unrolled_fold (sum) ---------------------------------
inline float unrolled_sum(const float* xs, size_t n) {
  float acc = 0.f, p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f, p4 = 0.f, p5 = 0.f, p6 = 0.f, p7 = 0.f;
  while (n >= 8) {
    p0 += xs[0]; p1 += xs[1]; p2 += xs[2]; p3 += xs[3];
    p4 += xs[4]; p5 += xs[5]; p6 += xs[6]; p7 += xs[7];
    xs += 8;
    n -= 8;
  }
  acc += (p0 + p4);
  acc += (p1 + p5);
  acc += (p2 + p6);
  acc += (p3 + p7);
  for (size_t i = 0; i < n && i < 7; ++i) acc += xs[i];
  return acc;
}

// compiler-rt __powisf2, which f32::powi lowers to.
inline float powi_f32(float a, int b) {
  const bool recip = b < 0;
  float r = 1.f;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.f / r : r;
}

// f32::max / f32::min ignore a NaN operand.
inline float fmax32(float a, float b) { return std::fmax(a, b); }
inline float fmin32(float a, float b) { return std::fmin(a, b); }

// Row-major strides of `shape` left-padded to `ndim`, with stride 0 where the
// dimension is broadcast (ndarray ArrayBase::broadcast).
inline std::vector<size_t> bcast_strides(const Shape& shape, const Shape& out) {
  size_t nd = out.size(), off = nd - shape.size();
  std::vector<size_t> st(nd, 0);
  size_t s = 1;
  for (size_t i = shape.size(); i-- > 0;) {
    st[i + off] = (shape[i] == 1 && out[i + off] != 1) ? 0 : s;
    s *= shape[i];
  }
  return st;
}

// Broadcast shape of two right-aligned shapes.
//  ndarray_operator = false: the rule of src/util.rs:2-26 and src/ops/cpu_ops.rs:319-335 (the larger
//    extent wins when one side is 1), followed by ndarray's `broadcast`, which only stretches
//    extents equal to 1 -- so pairing an extent 0 with an extent 1 is an IncompatibleShapes error.
//  ndarray_operator = true: ndarray's operator co-broadcast used by sub/div
//    (src/backend/cpu.rs:1259-1269): an extent 1 stretches to the other side, 0 included.
inline Shape broadcast_shapes(const Shape& a, const Shape& b, const char* op, bool ndarray_operator = false) {
  size_t nd = std::max(a.size(), b.size());
  Shape out(nd);
  for (size_t i = 0; i < nd; ++i) {
    size_t ad = i < nd - a.size() ? 1 : a[i - (nd - a.size())];
    size_t bd = i < nd - b.size() ? 1 : b[i - (nd - b.size())];
    if (ad == bd) out[i] = ad;
    else if (ad == 1 || bd == 1) {
      out[i] = ndarray_operator ? (ad == 1 ? bd : ad) : std::max(ad, bd);
      if (out[i] != ad && ad != 1) throw Error::incompatible(op, a, b);
      if (out[i] != bd && bd != 1) throw Error::incompatible(op, a, b);
    } else throw Error::incompatible(op, a, b);
  }
  return out;
}

template <class F>
Array broadcast_binary(const Array& a, const Array& b, const char* op, F f, bool ndarray_operator = false) {
  if (a.shape == b.shape) {
    Array out(std::vector<float>(a.size()), a.shape);
    for (size_t i = 0; i < a.size(); ++i) out.data[i] = f(a.data[i], b.data[i]);
    return out;
  }
  Shape os = broadcast_shapes(a.shape, b.shape, op, ndarray_operator);
  Array out(std::vector<float>(shape_numel(os)), os);
  auto sa = bcast_strides(a.shape, os), sb = bcast_strides(b.shape, os);
  size_t nd = os.size();
  std::vector<size_t> idx(nd, 0);
  size_t ia = 0, ib = 0;
  for (size_t o = 0; o < out.size(); ++o) {
    out.data[o] = f(a.data[ia], b.data[ib]);
    for (size_t d = nd; d-- > 0;) {
      idx[d]++;
      ia += sa[d];
      ib += sb[d];
      if (idx[d] < os[d]) break;
      ia -= sa[d] * os[d];
      ib -= sb[d] * os[d];
      idx[d] = 0;
    }
  }
  return out;
}

template <class F>
Array map(const Array& x, F f) {
  Array out(std::vector<float>(x.size()), x.shape);
  for (size_t i = 0; i < x.size(); ++i) out.data[i] = f(x.data[i]);
  return out;
}

// C[M,N] = A[M,K] * B[K,N], row-major, fp32 accumulation, sequential in k with fused
// multiply-add, as matrixmultiply's x86 FMA kernels do (stands in for
// matrixmultiply::sgemm; only the summation order differs).  All other arithmetic in
// this file is compiled with -ffp-contract=off, because Rust never contracts a*b+c.
inline void sgemm(size_t M, size_t N, size_t K, const float* A, const float* B, float* C) {
  constexpr size_t MR = 4, NR = 32;
  for (size_t i0 = 0; i0 < M; i0 += MR) {
    size_t mr = std::min(MR, M - i0);
    for (size_t j0 = 0; j0 < N; j0 += NR) {
      size_t nr = std::min(NR, N - j0);
      float acc[MR][NR];
      for (size_t i = 0; i < MR; ++i)
        for (size_t j = 0; j < NR; ++j) acc[i][j] = 0.f;
      if (mr == MR && nr == NR) {
        for (size_t k = 0; k < K; ++k) {
          const float* bk = B + k * N + j0;
          for (size_t i = 0; i < MR; ++i) {
            float a = A[(i0 + i) * K + k];
            for (size_t j = 0; j < NR; ++j) acc[i][j] = __builtin_fmaf(a, bk[j], acc[i][j]);
          }
        }
      } else {
        for (size_t k = 0; k < K; ++k) {
          const float* bk = B + k * N + j0;
          for (size_t i = 0; i < mr; ++i) {
            float a = A[(i0 + i) * K + k];
            for (size_t j = 0; j < nr; ++j) acc[i][j] = __builtin_fmaf(a, bk[j], acc[i][j]);
          }
        }
      }
      for (size_t i = 0; i < mr; ++i)
        for (size_t j = 0; j < nr; ++j) C[(i0 + i) * N + j0 + j] = acc[i][j];
    }
  }
}

inline std::vector<float> transpose2d(const float* x, size_t rows, size_t cols) {
  std::vector<float> t(rows * cols);
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) t[c * rows + r] = x[r * cols + c];
  return t;
}

struct CpuBackend {
  using Storage = Array;
  using OpB = Op<CpuBackend>;

  // ---- factories / shape access (src/backend/cpu.rs:129-242) -------------------
  // the gather loop of data::get_random_batch (src/data.rs:176-200): rows idx[i] of the flat host copy
  static Array gather_rows(const Array& x, size_t rows, size_t row_len, const std::vector<size_t>& idx) {
    Array out(std::vector<float>(idx.size() * row_len), Shape{idx.size(), row_len});
    for (size_t i = 0; i < idx.size(); ++i) {
      if (idx[i] >= rows || (idx[i] + 1) * row_len > x.data.size()) throw Error::internal("Index out of bounds accessing data slice");
      std::copy(x.data.begin() + idx[i] * row_len, x.data.begin() + (idx[i] + 1) * row_len, out.data.begin() + i * row_len);
    }
    return out;
  }
  static Array zeros(const Shape& s) { return Array::filled(s, 0.f); }
  // ---- random factories (src/backend/cpu.rs:133-194, src/init.rs:7-52) -------------------------------------------
  // rand's generator and distribution code are not part of the reference tree; what is restated here is the contract:
  // the distributions (U[low, high), N(mean, std^2), Bernoulli(p)), the empty-shape shortcuts and the parameter checks
  // (Uniform::new fails unless low < high and both are finite; Normal::new fails for a non-finite deviation;
  // Bernoulli::new fails unless 0 <= p <= 1).  std::mt19937_64 stands in for rand's ChaCha-based thread_rng.
  static std::mt19937_64& engine() {
    static std::mt19937_64 e{std::random_device{}()};
    return e;
  }
  static void manual_seed(uint64_t seed) { engine().seed(seed); }
  static Array random_uniform(const Shape& s, float low, float high) {
    if (shape_numel(s) == 0) return zeros(s);
    if (!(low < high) || !std::isfinite(low) || !std::isfinite(high) || !std::isfinite(high - low))
      throw Error(ErrorKind::InitializationError, "random_uniform: invalid range");
    Array a(std::vector<float>(shape_numel(s)), s);
    std::uniform_real_distribution<double> d(0.0, 1.0);
    for (auto& v : a.data) {
      float t = low + (high - low) * (float)d(engine());
      v = t < high ? t : std::nextafter(high, low);
    }
    return a;
  }
  static Array random_normal(const Shape& s, float mean, float std_dev) {
    if (shape_numel(s) == 0) return zeros(s);
    if (!std::isfinite(std_dev)) throw Error(ErrorKind::InitializationError, "random_normal: bad variance");
    Array a(std::vector<float>(shape_numel(s)), s);
    std::normal_distribution<double> d(0.0, 1.0);
    for (auto& v : a.data) v = mean + std_dev * (float)d(engine());
    return a;
  }
  static Array bernoulli(const Shape& s, float p) {
    if (shape_numel(s) == 0) return zeros(s);
    if (!(p >= 0.f && p <= 1.f)) throw Error(ErrorKind::InitializationError, "bernoulli: probability outside [0, 1]");
    Array a(std::vector<float>(shape_numel(s)), s);
    std::uniform_real_distribution<double> d(0.0, 1.0);
    for (auto& v : a.data) v = d(engine()) < (double)p ? 1.f : 0.f;
    return a;
  }
  static Array kaiming_uniform(size_t fan_in, const Shape& s) {  // src/init.rs:7-52
    if (s.empty()) throw Error::invalid_op("Cannot initialize tensor with empty shape");
    if (shape_numel(s) == 0) return zeros(s);
    if (fan_in == 0) throw Error::invalid_op("Fan-in cannot be zero for Kaiming initialization");
    const float bound = std::sqrt(6.0f / (float)fan_in);
    return random_uniform(s, -bound, bound);
  }
  static Array ones(const Shape& s) { return Array::filled(s, 1.f); }
  static Array from_vec(std::vector<float> v, const Shape& s) {
    if (v.size() != shape_numel(s)) throw Error::shape_mismatch(s, Shape{v.size()});  // src/array.rs:29-37
    return Array(std::move(v), s);
  }
  static const Shape& shape(const Array& a) { return a.shape; }
  static size_t size(const Array& a) { return a.size(); }
  static std::vector<float> copy_to_host(const Array& a) { return a.data; }
  static void update_from_host(Array& a, const std::vector<float>& d) {
    if (a.size() != d.size()) throw Error::shape_mismatch(a.shape, Shape{d.size()});
    a.data = d;
  }
  static void set_data(Array& a, Array d) { a = std::move(d); }
  // src/backend/cpu.rs:215-220 via src/array.rs:138-158
  static void set_shape(Array& a, const Shape& s) {
    if (shape_numel(s) != a.size()) throw Error::shape_mismatch(s, a.shape);
    a.shape = s;
  }
  static Array unused_grad(const Shape& s) { return zeros(s); }  // src/ops/mod.rs:362-364

  // ---- elementwise forward -----------------------------------------------------
  static Array mul(const Array& a, const Array& b) {  // src/ops/cpu_ops.rs:296-355
    return broadcast_binary(a, b, "mul", [](float x, float y) { return x * y; });
  }
  static Array add(const Array& a, const Array& b) {  // src/ops/cpu_ops.rs:358-416
    return broadcast_binary(a, b, "add", [](float x, float y) { return x + y; });
  }
  // src/backend/cpu.rs:1259-1269: ndarray operator broadcasting (the reference panics on
  // incompatible shapes; here that is an IncompatibleShapes error).
  static Array sub(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "sub", [](float x, float y) { return x - y; }, true);
  }
  static Array div(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "div", [](float x, float y) { return x / y; }, true);
  }
  static Array powf(const Array& a, const Array& b) {  // src/ops/cpu_ops.rs:765-830
    return broadcast_binary(a, b, "powf", [](float x, float y) { return std::pow(x, y); });
  }
  static Array maximum(const Array& a, const Array& b) {  // src/backend/cpu.rs:1817-1863
    return broadcast_binary(a, b, "maximum", [](float x, float y) { return fmax32(x, y); });
  }
  static Array minimum(const Array& a, const Array& b) {  // src/backend/cpu.rs:1944-1990
    return broadcast_binary(a, b, "minimum", [](float x, float y) { return fmin32(x, y); });
  }
  static Array equal(const Array& a, const Array& b) {  // src/backend/cpu.rs:684-722
    return broadcast_binary(a, b, "equal", [](float x, float y) { return std::fabs(x - y) < 1e-9f ? 1.f : 0.f; });
  }
  static Array not_equal(const Array& a, const Array& b) {  // src/backend/cpu.rs:860-898
    return broadcast_binary(a, b, "not_equal", [](float x, float y) { return std::fabs(x - y) >= 1e-9f ? 1.f : 0.f; });
  }
  static Array greater(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "greater", [](float x, float y) { return x > y ? 1.f : 0.f; });
  }
  static Array greater_equal(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "greater_equal", [](float x, float y) { return x >= y ? 1.f : 0.f; });
  }
  static Array less(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "less", [](float x, float y) { return x < y ? 1.f : 0.f; });
  }
  static Array less_equal(const Array& a, const Array& b) {
    return broadcast_binary(a, b, "less_equal", [](float x, float y) { return x <= y ? 1.f : 0.f; });
  }
  static Array div_scalar(const Array& x, float s) {  // src/backend/cpu.rs:1271-1279
    if (s == 0.0f) throw Error::invalid_op("Division by zero scalar");
    return map(x, [s](float v) { return v / s; });
  }
  static Array mul_scalar(const Array& x, float s) {  // src/backend/cpu.rs:1281-1283
    return map(x, [s](float v) { return v * s; });
  }
  static Array exp(const Array& x) { return map(x, [](float v) { return std::exp(v); }); }    // cpu.rs:1299
  static Array ln(const Array& x) { return map(x, [](float v) { return std::log(v); }); }     // cpu.rs:1304
  static Array abs(const Array& x) { return map(x, [](float v) { return std::fabs(v); }); }   // cpu.rs:1663
  static Array tanh(const Array& x) { return map(x, [](float v) { return std::tanh(v); }); }  // cpu.rs:1368
  static Array sin(const Array& x) { return map(x, [](float v) { return std::sin(v); }); }    // cpu.rs:2074
  static Array cos(const Array& x) { return map(x, [](float v) { return std::cos(v); }); }    // cpu.rs:2118
  static Array tan(const Array& x) { return map(x, [](float v) { return std::tan(v); }); }    // cpu.rs:2162
  static Array relu(const Array& x) { return map(x, [](float v) { return fmax32(v, 0.f); }); }  // cpu_ops.rs:444
  static Array sigmoid(const Array& x) {  // src/backend/cpu.rs:1689-1691
    return map(x, [](float v) { return 1.0f / (1.0f + std::exp(-v)); });
  }
  static Array softplus(const Array& x) {  // src/backend/cpu.rs:1737-1742 (naive ln(1+e^x))
    return map(x, [](float v) { return std::log(1.0f + std::exp(v)); });
  }
  static Array square(const Array& x) { return map(x, [](float v) { return v * v; }); }  // cpu.rs:1777-1791
  static Array sqrt(const Array& x) {                                                    // cpu.rs:1717-1723
    for (float v : x.data)
      if (v < 0.0f) throw Error::invalid_op("sqrt: input contains negative values");
    return map(x, [](float v) { return std::sqrt(v); });
  }
  static Array elu(const Array& x, float alpha) {  // src/backend/cpu.rs:1345-1361
    return map(x, [alpha](float v) { return v < 0.0f ? alpha * (std::exp(v) - 1.0f) : v; });
  }
  static Array clip(const Array& x, float lo, float hi) {  // src/backend/cpu.rs:2385-2393
    return map(x, [lo, hi](float v) { return fmin32(fmax32(v, lo), hi); });
  }

  // ---- layout ops ---------------------------------------------------------------
  static Array transpose(const Array& x) {  // src/backend/cpu.rs:1285-1292 (reverses all axes)
    if (x.ndim() <= 1) return x;
    if (x.ndim() == 2) return Array(transpose2d(x.data.data(), x.shape[0], x.shape[1]), Shape{x.shape[1], x.shape[0]});
    size_t nd = x.ndim();
    Shape os(x.shape.rbegin(), x.shape.rend());
    std::vector<size_t> in_st(nd);
    size_t s = 1;
    for (size_t i = nd; i-- > 0;) { in_st[i] = s; s *= x.shape[i]; }
    Array out(std::vector<float>(x.size()), os);
    std::vector<size_t> idx(nd, 0);
    for (size_t o = 0; o < out.size(); ++o) {
      size_t src = 0;
      for (size_t d = 0; d < nd; ++d) src += idx[d] * in_st[nd - 1 - d];
      out.data[o] = x.data[src];
      for (size_t d = nd; d-- > 0;) {
        if (++idx[d] < os[d]) break;
        idx[d] = 0;
      }
    }
    return out;
  }
  static Array broadcast_to(const Array& x, const Shape& shape) {  // src/array.rs:84-93
    if (shape.size() < x.ndim()) throw Error::incompatible("broadcast", x.shape, shape);
    size_t off = shape.size() - x.ndim();
    for (size_t i = 0; i < x.ndim(); ++i)
      if (x.shape[i] != shape[i + off] && x.shape[i] != 1) throw Error::incompatible("broadcast", x.shape, shape);
    Array out(std::vector<float>(shape_numel(shape)), shape);
    auto st = bcast_strides(x.shape, shape);
    size_t nd = shape.size();
    std::vector<size_t> idx(nd, 0);
    size_t src = 0;
    for (size_t o = 0; o < out.size(); ++o) {
      out.data[o] = x.data[src];
      for (size_t d = nd; d-- > 0;) {
        idx[d]++;
        src += st[d];
        if (idx[d] < shape[d]) break;
        src -= st[d] * shape[d];
        idx[d] = 0;
      }
    }
    return out;
  }
  static Array slice(const Array& x, const std::vector<Range>& ranges) {  // src/backend/cpu.rs:2207-2222
    if (ranges.size() != x.ndim()) throw Error::invalid_op("Slice ranges do not match input dimensionality");
    size_t nd = x.ndim();
    Shape os(nd);
    for (size_t i = 0; i < nd; ++i) os[i] = ranges[i].end - ranges[i].start;
    std::vector<size_t> st(nd);
    size_t s = 1;
    for (size_t i = nd; i-- > 0;) { st[i] = s; s *= x.shape[i]; }
    Array out(std::vector<float>(shape_numel(os)), os);
    std::vector<size_t> idx(nd, 0);
    for (size_t o = 0; o < out.size(); ++o) {
      size_t src = 0;
      for (size_t d = 0; d < nd; ++d) src += (idx[d] + ranges[d].start) * st[d];
      out.data[o] = x.data[src];
      for (size_t d = nd; d-- > 0;) {
        if (++idx[d] < os[d]) break;
        idx[d] = 0;
      }
    }
    return out;
  }
  static Array slice_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2225-2245
    if (op.op_type.kind != OpType::Slice) throw Error::internal("Incorrect OpType for slice_backward");
    const Shape& is = op.op_type.input_shape;
    const auto& ranges = op.op_type.ranges;
    size_t nd = is.size();
    Array out = zeros(is);
    std::vector<size_t> st(nd);
    size_t s = 1;
    for (size_t i = nd; i-- > 0;) { st[i] = s; s *= is[i]; }
    Shape gs(nd);
    for (size_t i = 0; i < nd; ++i) gs[i] = ranges[i].end - ranges[i].start;
    if (shape_numel(gs) != g.size()) throw Error::incompatible("slice_backward", gs, g.shape);
    std::vector<size_t> idx(nd, 0);
    for (size_t o = 0; o < g.size(); ++o) {
      size_t dst = 0;
      for (size_t d = 0; d < nd; ++d) dst += (idx[d] + ranges[d].start) * st[d];
      out.data[dst] = g.data[o];
      for (size_t d = nd; d-- > 0;) {
        if (++idx[d] < gs[d]) break;
        idx[d] = 0;
      }
    }
    return out;
  }
  static Array concat(const std::vector<const Array*>& xs, size_t axis) {  // src/backend/cpu.rs:2248-2261
    if (xs.empty()) throw Error::invalid_op("Cannot concat empty list of storages");
    Shape os = xs[0]->shape;
    if (axis >= os.size()) throw Error(ErrorKind::ShapeError, "ndarray::concatenate failed: axis out of bounds");
    size_t total = 0;
    for (auto* x : xs) {
      if (x->ndim() != os.size()) throw Error(ErrorKind::ShapeError, "ndarray::concatenate failed: incompatible shapes");
      for (size_t d = 0; d < os.size(); ++d)
        if (d != axis && x->shape[d] != os[d])
          throw Error(ErrorKind::ShapeError, "ndarray::concatenate failed: incompatible shapes");
      total += x->shape[axis];
    }
    os[axis] = total;
    size_t outer = 1, inner = 1;
    for (size_t d = 0; d < axis; ++d) outer *= os[d];
    for (size_t d = axis + 1; d < os.size(); ++d) inner *= os[d];
    Array out(std::vector<float>(shape_numel(os)), os);
    size_t off = 0;
    for (auto* x : xs) {
      size_t len = x->shape[axis] * inner;
      for (size_t o = 0; o < outer; ++o)
        std::memcpy(&out.data[o * total * inner + off], &x->data[o * len], len * sizeof(float));
      off += len;
    }
    return out;
  }
  static std::vector<Array> concat_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2264-2296
    if (op.op_type.kind != OpType::Concat) throw Error::internal("Incorrect OpType for concat_backward");
    size_t axis = *op.op_type.axis;
    std::vector<Array> grads;
    size_t off = 0;
    for (const Shape& s : op.op_type.input_shapes) {
      std::vector<Range> r;
      for (size_t d = 0; d < g.ndim(); ++d)
        r.push_back(d == axis ? Range{off, off + s[axis]} : Range{0, g.shape[d]});
      grads.push_back(slice(g, r));
      off += s[axis];
    }
    return grads;
  }
  static Array expand_dims(const Array& x, size_t axis) {  // src/backend/cpu.rs:2299-2313
    if (axis > x.ndim()) throw Error::invalid_index(axis);
    Array out = x;
    out.shape.insert(out.shape.begin() + axis, 1);
    return out;
  }
  static Array expand_dims_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2316-2340
    size_t axis = *op.op_type.axis;
    Shape orig = op.inputs[0].shape();
    Array out = g;
    if (axis < g.ndim() && g.shape[axis] == 1) {
      set_shape(out, orig);
    } else if (axis < g.ndim()) {
      out = sum_along_axis(g, axis);
      set_shape(out, orig);
    } else {
      throw Error::internal("expand_dims_backward: axis out of bounds for grad_output");
    }
    return out;
  }
  static Array squeeze(const Array& x, std::optional<size_t> axis) {  // src/backend/cpu.rs:2343-2368
    Shape ns;
    if (axis) {
      if (*axis >= x.ndim()) throw Error::invalid_index(*axis);
      if (x.shape[*axis] != 1) throw Error::invalid_op("Cannot squeeze axis (not size 1)");
      ns = x.shape;
      ns.erase(ns.begin() + *axis);
    } else {
      for (size_t d : x.shape)
        if (d != 1) ns.push_back(d);
    }
    Array out = x;
    set_shape(out, ns);
    return out;
  }
  static Array squeeze_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2371-2382
    Array out = g;
    set_shape(out, op.op_type.input_shape);
    return out;
  }

  // ---- reductions ---------------------------------------------------------------
  static void split_axis(const Shape& s, size_t axis, size_t& outer, size_t& len, size_t& inner) {
    outer = inner = 1;
    for (size_t d = 0; d < axis; ++d) outer *= s[d];
    len = s[axis];
    for (size_t d = axis + 1; d < s.size(); ++d) inner *= s[d];
  }
  static Shape remove_axis(const Shape& s, size_t axis) {
    Shape r = s;
    r.erase(r.begin() + axis);
    return r;
  }
  // src/array.rs:95-100 -> ndarray sum_axis: per-lane unrolled sum when the axis is
  // the contiguous one, otherwise `res = res + subview` for each index of the axis.
  static Array sum_along_axis(const Array& x, size_t axis) {
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    size_t outer, len, inner;
    split_axis(x.shape, axis, outer, len, inner);
    Array out = zeros(remove_axis(x.shape, axis));
    if (inner == 1) {
      for (size_t o = 0; o < outer; ++o) out.data[o] = unrolled_sum(&x.data[o * len], len);
    } else {
      for (size_t o = 0; o < outer; ++o)
        for (size_t k = 0; k < len; ++k) {
          const float* src = &x.data[(o * len + k) * inner];
          float* dst = &out.data[o * inner];
          for (size_t i = 0; i < inner; ++i) dst[i] = dst[i] + src[i];
        }
    }
    return out;
  }
  static float sum_all(const Array& x) { return unrolled_sum(x.data.data(), x.size()); }  // cpu.rs:1324-1327
  static Array sum_all_scalar(const Array& x) { return from_vec({sum_all(x)}, Shape{}); }  // ops/mod.rs:654-655
  static Array max_along_axis(const Array& x, size_t axis) {  // src/array.rs:102-109 (folds from f32::MIN)
    return fold_axis(x, axis, std::numeric_limits<float>::lowest(), fmax32);
  }
  template <class F>
  static Array fold_axis(const Array& x, size_t axis, float init, F f) {
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    size_t outer, len, inner;
    split_axis(x.shape, axis, outer, len, inner);
    Array out = Array::filled(remove_axis(x.shape, axis), init);
    for (size_t o = 0; o < outer; ++o)
      for (size_t k = 0; k < len; ++k)
        for (size_t i = 0; i < inner; ++i)
          out.data[o * inner + i] = f(out.data[o * inner + i], x.data[(o * len + k) * inner + i]);
    return out;
  }
  static Array mean(const Array& x, std::optional<size_t> axis) {  // src/ops/cpu_ops.rs:419-441
    if (axis) {
      if (*axis >= x.ndim()) throw Error::invalid_index(*axis);
      if (x.shape[*axis] == 0) throw Error::invalid_op("Mean failed along axis");
      Array s = sum_along_axis(x, *axis);
      float n = (float)x.shape[*axis];
      for (float& v : s.data) v = v / n;
      return s;
    }
    if (x.size() == 0) throw Error(ErrorKind::EmptyTensor, "empty tensor");
    return from_vec({sum_all(x) / (float)x.size()}, Shape{});
  }
  static Array max(const Array& x, std::optional<size_t> axis) {  // src/ops/cpu_ops.rs:486-507
    if (x.size() == 0) return zeros(x.shape);
    if (axis) return fold_axis(x, *axis, -INFINITY, fmax32);
    float m = -INFINITY;
    for (float v : x.data) m = fmax32(m, v);
    return from_vec({m}, Shape{});
  }
  static Array min(const Array& x, std::optional<size_t> axis) {  // src/ops/cpu_ops.rs:511-533
    if (x.size() == 0) return zeros(x.shape);
    if (axis) return fold_axis(x, *axis, INFINITY, fmin32);
    float m = INFINITY;
    for (float v : x.data) m = fmin32(m, v);
    return from_vec({m}, Shape{});
  }
  static Array prod(const Array& x, std::optional<size_t> axis) {  // src/ops/cpu_ops.rs:537-559
    if (x.size() == 0) return zeros(x.shape);
    if (axis) return fold_axis(x, *axis, 1.0f, [](float a, float b) { return a * b; });
    float p = 1.0f;
    for (float v : x.data) p *= v;
    return from_vec({p}, Shape{});
  }
  static Array logsumexp(const Array& x, std::optional<size_t> axis) {  // src/ops/cpu_ops.rs:564-597
    if (x.size() == 0) return zeros(x.shape);
    if (axis) {
      Array mx = fold_axis(x, *axis, -INFINITY, fmax32);
      Array shifted = sub(x, inserted(mx, *axis));
      Array e = exp(shifted);
      Array s = sum_along_axis(e, *axis);
      for (size_t i = 0; i < s.size(); ++i) s.data[i] = mx.data[i] + std::log(s.data[i]);
      return s;
    }
    float m = -INFINITY;
    for (float v : x.data) m = fmax32(m, v);
    Array e = map(x, [m](float v) { return std::exp(v - m); });
    return from_vec({m + std::log(sum_all(e))}, Shape{});
  }
  static Array inserted(const Array& x, size_t axis) {
    Array r = x;
    r.shape.insert(r.shape.begin() + axis, 1);
    return r;
  }
  static Array log_softmax(const Array& x, size_t axis) {  // src/ops/cpu_ops.rs:462-482
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    Array mx = fold_axis(x, axis, -INFINITY, fmax32);
    Array shifted = sub(x, inserted(mx, axis));
    Array e = exp(shifted);
    Array s = sum_along_axis(e, axis);
    Array lse = ln(s);
    return sub(shifted, inserted(lse, axis));
  }
  template <class Cmp>
  static Array arg_axis(const Array& x, size_t axis, float init, Cmp better) {
    if (x.size() == 0) return zeros(x.shape);
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    if (x.ndim() == 1) {
      size_t bi = 0;
      float bv = init;
      for (size_t i = 0; i < x.size(); ++i)
        if (better(x.data[i], bv)) { bv = x.data[i]; bi = i; }
      return from_vec({(float)bi}, Shape{});
    }
    size_t outer, len, inner;
    split_axis(x.shape, axis, outer, len, inner);
    Array out = zeros(remove_axis(x.shape, axis));
    for (size_t o = 0; o < outer; ++o)
      for (size_t i = 0; i < inner; ++i) {
        size_t bi = 0;
        float bv = init;
        for (size_t k = 0; k < len; ++k) {
          float v = x.data[(o * len + k) * inner + i];
          if (better(v, bv)) { bv = v; bi = k; }
        }
        out.data[o * inner + i] = (float)bi;
      }
    return out;
  }
  static Array argmax(const Array& x, size_t axis) {  // src/ops/cpu_ops.rs:601-679
    return arg_axis(x, axis, -INFINITY, [](float v, float b) { return v > b; });
  }
  static Array argmin(const Array& x, size_t axis) {  // src/ops/cpu_ops.rs:683-761
    return arg_axis(x, axis, INFINITY, [](float v, float b) { return v < b; });
  }

  // ---- matmul / conv / pool -----------------------------------------------------
  static Array matmul(const Array& a, const Array& b) {  // src/ops/cpu_ops.rs:64-85
    if (a.ndim() != 2) throw Error(ErrorKind::ShapeError, "Input 'a' is not 2D");
    if (b.ndim() != 2) throw Error(ErrorKind::ShapeError, "Input 'b' is not 2D");
    if (a.shape[1] != b.shape[0]) throw Error::incompatible("matmul", a.shape, b.shape);
    Array out(std::vector<float>(a.shape[0] * b.shape[1]), Shape{a.shape[0], b.shape[1]});
    sgemm(a.shape[0], b.shape[1], a.shape[1], a.data.data(), b.data.data(), out.data.data());
    return out;
  }

  static void im2col(const Array& input, size_t kh, size_t kw, Pair stride, Pair pad, size_t ho, size_t wo,
                     std::vector<float>& cols) {  // src/ops/cpu_ops.rs:111-142 / 199-230
    size_t n = input.shape[0], c = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t ckk = c * kh * kw, hw = ho * wo;
    cols.assign(n * ckk * hw, 0.f);
    for (size_t b = 0; b < n; ++b) {
      const float* img = &input.data[b * c * h * w];
      float* col = &cols[b * ckk * hw];
      size_t col_idx = 0;
      for (size_t y = 0; y < ho; ++y)
        for (size_t x = 0; x < wo; ++x) {
          long ys = (long)(y * stride.first) - (long)pad.first, xs = (long)(x * stride.second) - (long)pad.second;
          size_t i = 0;
          for (size_t ch = 0; ch < c; ++ch)
            for (size_t ky = 0; ky < kh; ++ky)
              for (size_t kx = 0; kx < kw; ++kx) {
                long iy = ys + (long)ky, ix = xs + (long)kx;
                float v = (iy >= 0 && (size_t)iy < h && ix >= 0 && (size_t)ix < w) ? img[(ch * h + iy) * w + ix] : 0.f;
                col[i * hw + col_idx] = v;
                ++i;
              }
          ++col_idx;
        }
    }
  }

  static Array conv2d(const Array& input, const Array& weights, const Array* bias, Pair stride,
                      Pair pad) {  // src/ops/cpu_ops.rs:88-178
    if (input.ndim() != 4 || weights.ndim() != 4) throw Error::invalid_op("conv2d expects 4D input and weights");
    size_t n = input.shape[0], cin = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t cout = weights.shape[0], kh = weights.shape[2], kw = weights.shape[3];
    if (cin != weights.shape[1]) throw Error::invalid_op("conv2d: input channels != weight channels");
    size_t ho = (h + 2 * pad.first - kh) / stride.first + 1, wo = (w + 2 * pad.second - kw) / stride.second + 1;
    size_t ckk = cin * kh * kw, hw = ho * wo;
    std::vector<float> cols;
    im2col(input, kh, kw, stride, pad, ho, wo, cols);
    Array out(std::vector<float>(n * cout * hw), Shape{n, cout, ho, wo});
    for (size_t b = 0; b < n; ++b)
      sgemm(cout, hw, ckk, weights.data.data(), &cols[b * ckk * hw], &out.data[b * cout * hw]);
    if (bias) {
      if (bias->size() != cout) throw Error::invalid_op("conv2d: bias shape mismatch");
      for (size_t b = 0; b < n; ++b)
        for (size_t co = 0; co < cout; ++co)
          for (size_t i = 0; i < hw; ++i) out.data[(b * cout + co) * hw + i] += bias->data[co];
    }
    return out;
  }

  // src/ops/cpu_ops.rs:181-293.  The need_* flags exist for interface parity with
  // the CUDA backend and are ignored: the reference always computes all three.
  static std::tuple<Array, Array, std::optional<Array>> conv2d_backward(const Array& input, const Array& weights,
                                                                        const Array& grad_output, Pair stride,
                                                                        Pair pad, bool = true, bool = true,
                                                                        bool = true) {
    size_t n = input.shape[0], cin = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t cout = weights.shape[0], kh = weights.shape[2], kw = weights.shape[3];
    size_t ho = (h + 2 * pad.first - kh) / stride.first + 1, wo = (w + 2 * pad.second - kw) / stride.second + 1;
    size_t ckk = cin * kh * kw, hw = ho * wo;
    if (grad_output.size() != n * cout * hw)
      throw Error::shape_mismatch(Shape{n, cout, ho, wo}, grad_output.shape);
    std::vector<float> cols;
    im2col(input, kh, kw, stride, pad, ho, wo, cols);
    // dW = sum_b grad_out[b] . cols[b]^T, accumulated sample by sample (:244-250)
    std::vector<float> grad_w(cout * ckk, 0.f), tmp(cout * ckk);
    for (size_t b = 0; b < n; ++b) {
      std::vector<float> colt = transpose2d(&cols[b * ckk * hw], ckk, hw);  // [hw, ckk]
      sgemm(cout, ckk, hw, &grad_output.data[b * cout * hw], colt.data(), tmp.data());
      for (size_t i = 0; i < grad_w.size(); ++i) grad_w[i] = grad_w[i] + tmp[i];
    }
    // db (:252-257)
    std::vector<float> grad_b(cout, 0.f);
    for (size_t b = 0; b < n; ++b)
      for (size_t co = 0; co < cout; ++co) grad_b[co] += unrolled_sum(&grad_output.data[(b * cout + co) * hw], hw);
    // dX: grad_cols = W2d^T . grad_out[b], then col2im (:259-287)
    std::vector<float> grad_in(n * cin * h * w, 0.f);
    std::vector<float> wt = transpose2d(weights.data.data(), cout, ckk);  // [ckk, cout]
    std::vector<float> grad_cols(ckk * hw);
    const bool faithful = conv_dx_faithful();
    for (size_t b = 0; b < n; ++b) {
      sgemm(ckk, hw, cout, wt.data(), &grad_output.data[b * cout * hw], grad_cols.data());
      size_t pix = 0;
      for (size_t y = 0; y < ho; ++y)
        for (size_t x = 0; x < wo; ++x, ++pix) {
          long ys = (long)(y * stride.first) - (long)pad.first, xs = (long)(x * stride.second) - (long)pad.second;
          size_t col_idx = faithful ? 0 : pix;
          size_t i = 0;
          for (size_t ch = 0; ch < cin; ++ch)
            for (size_t ky = 0; ky < kh; ++ky)
              for (size_t kx = 0; kx < kw; ++kx) {
                long iy = ys + (long)ky, ix = xs + (long)kx;
                if (iy >= 0 && iy < (long)h && ix >= 0 && ix < (long)w)
                  grad_in[((b * cin + ch) * h + iy) * w + ix] += grad_cols[i * hw + col_idx];
                ++i;
              }
        }
    }
    return {Array(std::move(grad_in), input.shape), Array(std::move(grad_w), weights.shape),
            std::optional<Array>(Array(std::move(grad_b), Shape{cout}))};
  }

  // src/backend/cpu.rs:974-1091.  Output coordinates are computed in unsigned
  // arithmetic (`h_in*stride + kh - padding`), so a negative position wraps to a huge
  // value and fails the `< output_height` test, exactly as in a release build of the
  // reference.
  static Array conv2d_transpose(const Array& input, const Array& weights, const Array* bias, Pair stride, Pair pad) {
    if (input.ndim() != 4) throw Error(ErrorKind::ShapeError, "Expected 4D input tensor for conv2d_transpose");
    if (weights.ndim() != 4) throw Error(ErrorKind::ShapeError, "Expected 4D weights tensor for conv2d_transpose");
    size_t n = input.shape[0], cin = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t cout = weights.shape[1], kh = weights.shape[2], kw = weights.shape[3];
    if (cin != weights.shape[0]) throw Error::shape_mismatch(Shape{n, weights.shape[0], h, w}, input.shape);
    if (bias && (bias->ndim() != 1 || bias->shape[0] != cout)) throw Error::shape_mismatch(Shape{cout}, bias->shape);
    size_t oh = (h - 1) * stride.first + kh - 2 * pad.first, ow = (w - 1) * stride.second + kw - 2 * pad.second;
    Array out = zeros(Shape{n, cout, oh, ow});
    for (size_t b = 0; b < n; ++b)
      for (size_t oc = 0; oc < cout; ++oc) {
        float* o = &out.data[(b * cout + oc) * oh * ow];
        for (size_t ic = 0; ic < cin; ++ic)
          for (size_t hi = 0; hi < h; ++hi)
            for (size_t wi = 0; wi < w; ++wi) {
              float iv = input.data[((b * cin + ic) * h + hi) * w + wi];
              for (size_t ky = 0; ky < kh; ++ky)
                for (size_t kx = 0; kx < kw; ++kx) {
                  size_t y = hi * stride.first + ky - pad.first, x = wi * stride.second + kx - pad.second;
                  if (y < oh && x < ow) o[y * ow + x] += iv * weights.data[((ic * cout + oc) * kh + ky) * kw + kx];
                }
            }
        if (bias)
          for (size_t i = 0; i < oh * ow; ++i) o[i] += bias->data[oc];
      }
    return out;
  }

  // src/backend/cpu.rs:1093-1246
  static std::tuple<Array, Array, std::optional<Array>> conv2d_transpose_backward(const Array& input,
                                                                                  const Array& weights,
                                                                                  const Array& g, Pair stride,
                                                                                  Pair pad, bool = true,
                                                                                  bool = true, bool = true) {
    if (input.ndim() != 4 || weights.ndim() != 4 || g.ndim() != 4)
      throw Error(ErrorKind::ShapeError, "Expected 4D tensors for conv2d_transpose_backward");
    size_t n = input.shape[0], cin = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t cout = weights.shape[1], kh = weights.shape[2], kw = weights.shape[3];
    size_t oh = g.shape[2], ow = g.shape[3];
    if (cin != weights.shape[0]) throw Error::shape_mismatch(Shape{n, weights.shape[0], h, w}, input.shape);
    if (g.shape[1] != cout) throw Error::shape_mismatch(Shape{n, cout, oh, ow}, g.shape);
    Array gi = zeros(input.shape), gw = zeros(weights.shape);
    for (size_t b = 0; b < n; ++b)
      for (size_t ic = 0; ic < cin; ++ic)
        for (size_t hi = 0; hi < h; ++hi)
          for (size_t wi = 0; wi < w; ++wi) {
            float& acc = gi.data[((b * cin + ic) * h + hi) * w + wi];
            for (size_t oc = 0; oc < cout; ++oc)
              for (size_t ky = 0; ky < kh; ++ky)
                for (size_t kx = 0; kx < kw; ++kx) {
                  size_t y = hi * stride.first + ky - pad.first, x = wi * stride.second + kx - pad.second;
                  if (y < oh && x < ow)
                    acc += g.data[((b * cout + oc) * oh + y) * ow + x] *
                           weights.data[((ic * cout + oc) * kh + ky) * kw + kx];
                }
          }
    for (size_t ic = 0; ic < cin; ++ic)
      for (size_t oc = 0; oc < cout; ++oc)
        for (size_t ky = 0; ky < kh; ++ky)
          for (size_t kx = 0; kx < kw; ++kx) {
            float acc = 0.f;
            for (size_t b = 0; b < n; ++b)
              for (size_t hi = 0; hi < h; ++hi)
                for (size_t wi = 0; wi < w; ++wi) {
                  size_t y = hi * stride.first + ky - pad.first, x = wi * stride.second + kx - pad.second;
                  if (y < oh && x < ow)
                    acc += input.data[((b * cin + ic) * h + hi) * w + wi] * g.data[((b * cout + oc) * oh + y) * ow + x];
                }
            gw.data[((ic * cout + oc) * kh + ky) * kw + kx] = acc;
          }
    std::optional<Array> gb;
    if (cout > 0) {
      gb = zeros(Shape{cout});
      for (size_t oc = 0; oc < cout; ++oc) {
        float acc = 0.f;
        for (size_t b = 0; b < n; ++b)
          for (size_t i = 0; i < oh * ow; ++i) acc += g.data[(b * cout + oc) * oh * ow + i];
        gb->data[oc] = acc;
      }
    }
    return {std::move(gi), std::move(gw), std::move(gb)};
  }

  // src/ops/cpu_ops.rs:7-61: first maximum wins in (ky,kx) scan order, strict `>`,
  // padding reads as -inf, the in-window index is stored as f32.
  static std::pair<Array, Array> max_pool2d(const Array& input, Pair k, Pair s, Pair p) {
    if (input.ndim() != 4) throw Error::invalid_op("max_pool2d expects 4D input (NCHW)");
    size_t n = input.shape[0], c = input.shape[1], h = input.shape[2], w = input.shape[3];
    size_t ho = (h + 2 * p.first - k.first) / s.first + 1, wo = (w + 2 * p.second - k.second) / s.second + 1;
    Array out = zeros(Shape{n, c, ho, wo}), idx = zeros(Shape{n, c, ho, wo});
    for (size_t bc = 0; bc < n * c; ++bc)
      for (size_t y = 0; y < ho; ++y)
        for (size_t x = 0; x < wo; ++x) {
          float mv = -INFINITY;
          size_t mi = 0, iw = 0;
          for (size_t ky = 0; ky < k.first; ++ky)
            for (size_t kx = 0; kx < k.second; ++kx) {
              long iy = (long)(y * s.first + ky) - (long)p.first, ix = (long)(x * s.second + kx) - (long)p.second;
              float v = (iy >= 0 && iy < (long)h && ix >= 0 && ix < (long)w) ? input.data[(bc * h + iy) * w + ix] : -INFINITY;
              if (v > mv) { mv = v; mi = iw; }
              ++iw;
            }
          out.data[(bc * ho + y) * wo + x] = mv;
          idx.data[(bc * ho + y) * wo + x] = (float)mi;
        }
    return {std::move(out), std::move(idx)};
  }
  // src/backend/cpu.rs:915-948 -> src/ops/cpu_backward.rs:9-46
  static Array max_pool2d_backward(const OpB& op, const Array& g) {
    if (op.inputs.size() < 2) throw Error::invalid_op("max_pool2d_backward requires at least 2 inputs (input and indices)");
    if (op.op_type.kind != OpType::MaxPool2D) throw Error::internal("Expected MaxPool2d op type for max_pool2d_backward");
    Shape is = op.inputs[0].shape();
    const Array& idx = op.inputs[1].data();
    Pair k = op.op_type.kernel_size, s = op.op_type.stride, p = op.op_type.padding;
    size_t n = is[0], c = is[1], h = is[2], w = is[3];
    size_t ho = (h + 2 * p.first - k.first) / s.first + 1, wo = (w + 2 * p.second - k.second) / s.second + 1;
    Array gi = zeros(is);
    for (size_t bc = 0; bc < n * c; ++bc)
      for (size_t y = 0; y < ho; ++y)
        for (size_t x = 0; x < wo; ++x) {
          size_t o = (bc * ho + y) * wo + x;
          float gv = o < g.size() ? g.data[o] : 0.f;
          size_t flat = (size_t)std::lround(o < idx.size() ? idx.data[o] : 0.f);
          size_t ky = flat / k.second, kx = flat % k.second;
          long iy = (long)(y * s.first + ky) - (long)p.first, ix = (long)(x * s.second + kx) - (long)p.second;
          if (iy >= 0 && iy < (long)h && ix >= 0 && ix < (long)w) gi.data[(bc * h + iy) * w + ix] += gv;
        }
    return gi;
  }

  // ---- backward: generic helpers of src/ops/cpu_backward.rs ---------------------
  // src/ops/cpu_backward.rs:523-678
  static Array unbroadcast(Array grad, const Shape& target) {
    if (grad.shape == target) return grad;
    Array cur = std::move(grad);
    size_t gnd = cur.ndim(), tnd = target.size();
    Shape cur_shape = cur.shape;
    if (gnd > tnd) {
      for (size_t axis = gnd - tnd; axis-- > 0;) {
        cur = sum_along_axis(cur, axis);
        if (axis < cur_shape.size()) cur_shape.erase(cur_shape.begin() + axis);
      }
    }
    size_t cnd = cur_shape.size();
    size_t pad_len = tnd > cnd ? tnd - cnd : 0;
    std::vector<size_t> axes;
    for (size_t i = 0; i < tnd; ++i) {
      size_t cd = i < pad_len ? 1 : cur_shape[i - pad_len];
      if (target[i] == 1 && cd != 1) {
        size_t ai = i > pad_len ? i - pad_len : 0;
        if (ai < cnd) axes.push_back(ai);
      }
    }
    std::sort(axes.begin(), axes.end(), std::greater<size_t>());
    axes.erase(std::unique(axes.begin(), axes.end()), axes.end());
    for (size_t axis : axes)
      if (axis < cur.ndim()) cur = sum_along_axis(cur, axis);
    if (cur.shape == target) return cur;
    size_t fs = std::max<size_t>(shape_numel(cur.shape), 1), ts = std::max<size_t>(shape_numel(target), 1);
    if (fs == ts) {
      try {
        set_shape(cur, target);
      } catch (const Error& e) {
        throw Error::internal(std::string("unbroadcast: Failed final reshape: ") + e.what());
      }
      return cur;
    }
    throw Error::incompatible("unbroadcast (final shape/size)", cur.shape, target);
  }

  static std::pair<Array, Array> matmul_backward(const OpB& op, const Array& g) {  // cpu_backward.rs:110-133
    if (op.inputs.size() != 2) throw Error::invalid_op("Matmul requires 2 inputs");
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array bt = transpose(b);
    Array ga = matmul(g, bt);
    Array at = transpose(a);
    Array gb = matmul(at, g);
    return {std::move(ga), std::move(gb)};
  }
  // src/ops/mod.rs:161-175: the closure attached by ops::matmul (same math).
  static std::pair<Array, Array> matmul_closure_backward(const OpB& op, const Array& g) {
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array bt = transpose(b);
    Array at = transpose(a);
    Array ga = matmul(g, bt);
    Array gb = matmul(at, g);
    return {std::move(ga), std::move(gb)};
  }
  static std::pair<Array, Array> mul_backward(const OpB& op, const Array& g) {  // cpu_backward.rs:136-160
    if (op.inputs.size() != 2) throw Error::invalid_op("Mul requires 2 inputs");
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array ga = mul(g, b), gb = mul(g, a);
    return {unbroadcast(std::move(ga), a.shape), unbroadcast(std::move(gb), b.shape)};
  }
  static std::pair<Array, Array> add_backward(const OpB& op, const Array& g) {  // cpu_backward.rs:163-184
    if (op.inputs.size() != 2) throw Error::invalid_op("Add requires 2 inputs");
    Array ga = g, gb = g;
    return {unbroadcast(std::move(ga), op.inputs[0].data().shape), unbroadcast(std::move(gb), op.inputs[1].data().shape)};
  }
  // src/backend/cpu.rs:1617-1632.  The reference CPU code returns the two gradients
  // un-reduced; its CUDA differential tests (tests/ops_cuda_backward_tests.rs:1041-1175)
  // pin that a broadcast operand's gradient is summed back to the operand's shape, and
  // add_grad would reject the un-reduced shape.  The reduction is applied here so that
  // broadcast sub/div have a usable expected value; same-shape operands are unaffected.
  static std::pair<Array, Array> sub_backward(const OpB& op, const Array& g) {
    if (op.inputs.size() != 2) throw Error::invalid_op("Sub requires 2 inputs");
    Array ga = g;
    Array gb = div_scalar(g, -1.0f);
    return {unbroadcast(std::move(ga), op.inputs[0].data().shape), unbroadcast(std::move(gb), op.inputs[1].data().shape)};
  }
  static std::pair<Array, Array> div_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1592-1615
    if (op.inputs.size() != 2) throw Error::invalid_op("Div requires 2 inputs");
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array recip = div(ones(b.shape), b);
    Array b2 = mul(b, b);
    Array neg = div_scalar(div(a, b2), -1.0f);
    Array ga = mul(g, recip), gb = mul(g, neg);
    return {unbroadcast(std::move(ga), a.shape), unbroadcast(std::move(gb), b.shape)};
  }
  static std::pair<Array, Array> powf_backward(const OpB& op, const Array& g) {  // cpu_backward.rs:467-520
    if (op.inputs.size() != 2) throw Error::invalid_op("powf_backward expects 2 inputs");
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array apb = powf(a, b);
    Array one = broadcast_to(from_vec({1.0f}, Shape{}), b.shape);
    Array bm1 = sub(b, one);
    Array apbm1 = powf(a, bm1);
    Array t = mul(b, apbm1);
    Array ga = mul(g, t);
    Array lna = ln(a);
    Array t2 = mul(apb, lna);
    Array gb = mul(g, t2);
    return {unbroadcast(std::move(ga), a.shape), unbroadcast(std::move(gb), b.shape)};
  }
  static std::pair<Array, Array> maximum_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1865-1942
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array ma = broadcast_binary(a, b, "maximum_backward", [](float x, float y) { return x >= y ? 1.f : 0.f; });
    Array mb = broadcast_binary(a, b, "maximum_backward", [](float x, float y) { return y > x ? 1.f : 0.f; });
    Array gbc = broadcast_to(g, ma.shape);
    return {unbroadcast(mul(gbc, ma), a.shape), unbroadcast(mul(gbc, mb), b.shape)};
  }
  static std::pair<Array, Array> minimum_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1992-2071
    const Array& a = op.inputs[0].data();
    const Array& b = op.inputs[1].data();
    Array ma = broadcast_binary(a, b, "minimum_backward", [](float x, float y) { return x <= y ? 1.f : 0.f; });
    Array mb = broadcast_binary(a, b, "minimum_backward", [](float x, float y) { return y < x ? 1.f : 0.f; });
    Array gbc = broadcast_to(g, ma.shape);
    return {unbroadcast(mul(gbc, ma), a.shape), unbroadcast(mul(gbc, mb), b.shape)};
  }

  // Broadcast a reduced gradient back over `axis` (or over everything).
  static Array expand_reduced(const Array& r, std::optional<size_t> axis, const Shape& in_shape) {
    if (!axis) return broadcast_to(r, in_shape);
    if (*axis >= in_shape.size()) throw Error::invalid_index(*axis);
    return broadcast_to(inserted(r, *axis), in_shape);
  }
  static Array sum_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1455-1510
    if (op.inputs.size() != 1) throw Error::invalid_op("Sum backward expects 1 input");
    Shape is = op.inputs[0].shape();
    if (op.op_type.kind != OpType::Sum) throw Error::internal("Incorrect OpType for sum_backward");
    if (!op.op_type.axis) {
      if (!g.shape.empty()) throw Error::shape_mismatch(Shape{}, g.shape);
      return Array::filled(is, g.data.at(0));
    }
    if (*op.op_type.axis >= is.size()) throw Error::invalid_index(*op.op_type.axis);
    return broadcast_to(inserted(g, *op.op_type.axis), is);
  }
  static Array mean_backward(const OpB& op, const Array& g) {  // src/ops/cpu_backward.rs:681-780
    if (op.inputs.size() != 1) throw Error::invalid_op("Mean requires 1 input");
    const Array& x = op.inputs[0].data();
    if (op.op_type.kind != OpType::Mean) throw Error::internal("Incorrect OpType passed to mean_backward");
    if (!op.op_type.axis) {
      float size = (float)std::max<size_t>(x.size(), 1);
      return div_scalar(broadcast_to(g, x.shape), size);
    }
    size_t axis = *op.op_type.axis;
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    float n = (float)std::max<size_t>(x.shape[axis], 1);
    if (axis > g.ndim()) throw Error::invalid_index(axis);
    return div_scalar(broadcast_to(inserted(g, axis), x.shape), n);
  }
  static Array extremum_backward(const OpB& op, const Array& g, bool is_max) {  // cpu.rs:342-433 / 435-548
    if (op.inputs.size() != 1) throw Error::invalid_op("max/min_backward expects 1 input");
    const Array& x = op.inputs[0].data();
    auto axis = op.op_type.axis;
    Array ext = is_max ? max(x, axis) : min(x, axis);
    Array ext_b = expand_reduced(ext, axis, x.shape);
    Array mask = equal(x, ext_b);
    Array count = axis ? sum_along_axis(mask, *axis) : from_vec({sum_all(mask)}, Shape{});
    Array count_b = expand_reduced(count, axis, x.shape);
    Array g_b = expand_reduced(g, axis, x.shape);
    Array safe = add(count_b, broadcast_to(from_vec({1e-9f}, Shape{}), x.shape));
    return div(mul(g_b, mask), safe);
  }
  static Array max_backward(const OpB& op, const Array& g) { return extremum_backward(op, g, true); }
  static Array min_backward(const OpB& op, const Array& g) { return extremum_backward(op, g, false); }
  static Array prod_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:550-613
    if (op.inputs.size() != 1) throw Error::invalid_op("prod_backward expects 1 input");
    const Array& x = op.inputs[0].data();
    auto axis = op.op_type.axis;
    Array p_b = expand_reduced(prod(x, axis), axis, x.shape);
    Array g_b = expand_reduced(g, axis, x.shape);
    Array safe = add(x, broadcast_to(from_vec({1e-10f}, Shape{}), x.shape));
    return div(mul(g_b, p_b), safe);
  }
  static Array logsumexp_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:615-680
    if (op.inputs.size() != 1) throw Error::invalid_op("logsumexp_backward expects 1 input");
    const Array& x = op.inputs[0].data();
    auto axis = op.op_type.axis;
    Array lse_b = expand_reduced(logsumexp(x, axis), axis, x.shape);
    Array g_b = expand_reduced(g, axis, x.shape);
    Array softmax = exp(sub(x, lse_b));
    return mul(g_b, softmax);
  }
  static Array log_softmax_backward(const OpB& op, const Array& g) {  // src/ops/cpu_backward.rs:801-845
    if (op.inputs.empty()) throw Error::invalid_op("LogSoftmax requires 1 input");
    const Array& x = op.inputs[0].data();
    size_t axis = *op.op_type.axis;
    Array y = log_softmax(x, axis);
    Array p = exp(y);
    Array sg = sum_along_axis(g, axis);
    if (axis >= x.ndim()) throw Error::invalid_index(axis);
    Array sg_b = broadcast_to(inserted(sg, axis), x.shape);
    return sub(g, mul(p, sg_b));
  }
  static Array relu_backward(const OpB& op, const Array& g) {  // cpu_backward.rs:783-798 (mask is x > 0)
    if (op.inputs.size() != 1) throw Error::invalid_op("Relu requires 1 input");
    Array mask = map(op.inputs[0].data(), [](float v) { return v > 0.0f ? 1.0f : 0.0f; });
    return mul(g, mask);
  }
  static Array elu_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1525-1575
    if (op.inputs.size() != 1) throw Error::invalid_op("ELU backward expects 1 input");
    float alpha = op.op_type.scalar;
    const Array& x = op.inputs[0].data();
    if (x.shape != g.shape) throw Error::shape_mismatch(x.shape, g.shape);
    Array out(std::vector<float>(x.size()), x.shape);
    for (size_t i = 0; i < x.size(); ++i) {
      float d = x.data[i] < 0.0f ? alpha * std::exp(x.data[i]) : 1.0f;
      out.data[i] = g.data[i] * d;
    }
    return out;
  }
  static Array exp_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1634-1646
    return mul(g, exp(op.inputs.at(0).data()));
  }
  static Array ln_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1648-1661
    const Array& x = op.inputs.at(0).data();
    return mul(g, div(ones(x.shape), x));
  }
  static Array abs_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1667-1687
    Array sign = map(op.inputs.at(0).data(), [](float v) { return v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f); });
    return mul(g, sign);
  }
  static Array sigmoid_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1693-1715
    Array y = sigmoid(op.inputs.at(0).data());
    Array d = mul(y, sub(ones(y.shape), y));
    return mul(g, d);
  }
  static Array tanh_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1372-1394
    Array y = tanh(op.inputs.at(0).data());
    Array d = sub(ones(y.shape), mul(y, y));
    return mul(g, d);
  }
  static Array sqrt_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1725-1735
    Array h = map(op.inputs.at(0).data(), [](float v) { return 0.5f / std::sqrt(v); });
    return broadcast_binary(g, h, "sqrt_backward", [](float a, float b) { return a * b; });
  }
  static Array softplus_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1744-1762
    Array d = map(op.inputs.at(0).data(), [](float v) { return 1.0f / (1.0f + std::exp(-v)); });
    return mul(g, d);
  }
  static Array square_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:1793-1815
    if (op.inputs.size() != 1) throw Error::invalid_op("square_backward expects 1 input");
    Array two_x = map(op.inputs[0].data(), [](float v) { return 2.0f * v; });
    return mul(g, two_x);
  }
  static Array sin_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2089-2115
    if (op.inputs.size() != 1) throw Error::internal("sin_backward expects 1 input");
    const Array& x = op.inputs[0].data();
    if (x.shape != g.shape) throw Error::shape_mismatch(x.shape, g.shape);
    Array out(std::vector<float>(x.size()), x.shape);
    for (size_t i = 0; i < x.size(); ++i) out.data[i] = std::cos(x.data[i]) * g.data[i];
    return out;
  }
  static Array cos_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2133-2159: -sin(x) * g
    if (op.inputs.size() != 1) throw Error::internal("cos_backward expects 1 input");
    const Array& x = op.inputs[0].data();
    if (x.shape != g.shape) throw Error::shape_mismatch(x.shape, g.shape);
    Array out(std::vector<float>(x.size()), x.shape);
    for (size_t i = 0; i < x.size(); ++i) out.data[i] = -std::sin(x.data[i]) * g.data[i];
    return out;
  }
  static Array tan_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2177-2202: g * (1 / (cos x * cos x))
    if (op.inputs.size() != 1) throw Error::internal("tan_backward expects 1 input");
    Array c = cos(op.inputs[0].data());
    Array c2 = mul(c, c);
    Array d = div(ones(c2.shape), c2);
    return mul(g, d);
  }
  static Array clip_backward(const OpB& op, const Array& g) {  // src/backend/cpu.rs:2396-2413
    float lo = op.op_type.min_val, hi = op.op_type.max_val;
    Array mask = map(op.inputs.at(0).data(), [lo, hi](float v) { return (v >= lo && v <= hi) ? 1.0f : 0.0f; });
    return broadcast_binary(g, mask, "clip_backward", [](float a, float b) { return a * b; });
  }

  // ---- optimizer steps ----------------------------------------------------------
  static void check3(const Array& p, const Array& a, const Array& b) {
    if (p.shape != a.shape) throw Error::shape_mismatch(p.shape, a.shape);
    if (p.shape != b.shape) throw Error::shape_mismatch(p.shape, b.shape);
  }
  static void sgd_step(Array& w, const Array& dw, float lr) {  // src/backend/cpu.rs:244-260
    if (w.shape != dw.shape) throw Error::shape_mismatch(w.shape, dw.shape);
    for (size_t i = 0; i < w.size(); ++i) w.data[i] -= lr * dw.data[i];
  }
  static void momentum_sgd_step(Array& p, const Array& g, Array& vel, float lr, float mu) {  // cpu.rs:81-126
    if (p.shape != vel.shape) throw Error::shape_mismatch(p.shape, vel.shape);
    if (p.shape != g.shape) throw Error::shape_mismatch(p.shape, g.shape);
    for (size_t i = 0; i < p.size(); ++i) {
      vel.data[i] = mu * vel.data[i] + g.data[i];
      p.data[i] -= lr * vel.data[i];
    }
  }
  static void adagrad_step(Array& p, const Array& g, Array& acc, float lr, float eps) {  // cpu.rs:32-78
    check3(p, g, acc);
    for (size_t i = 0; i < p.size(); ++i) {
      acc.data[i] += g.data[i] * g.data[i];
      p.data[i] -= lr * g.data[i] / (std::sqrt(acc.data[i]) + eps);
    }
  }
  static void adam_step(Array& p, const Array& g, Array& m, Array& v, float lr, float b1, float b2, float eps,
                        size_t t) {  // src/backend/cpu.rs:262-318
    check3(p, g, m);
    if (p.shape != v.shape) throw Error::shape_mismatch(p.shape, v.shape);
    if (t == 0) throw Error::internal("Adam step called with t=0");
    float bc1 = 1.0f - powi_f32(b1, (int)t), bc2 = 1.0f - powi_f32(b2, (int)t);
    for (size_t i = 0; i < p.size(); ++i) {
      float gi = g.data[i];
      m.data[i] = b1 * m.data[i] + (1.0f - b1) * gi;
      v.data[i] = b2 * v.data[i] + (1.0f - b2) * (gi * gi);
      float mh = m.data[i] / bc1, vh = v.data[i] / bc2;
      p.data[i] -= lr * mh / (std::sqrt(vh) + eps);
    }
  }
};

}  // namespace oracle
