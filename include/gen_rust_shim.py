#!/usr/bin/env python
"""Writes include/b200_backend.rs: the Rust side of include/rt_b200.h for the reference crate.

Two parts:
  * `mod ffi`: one `extern "C"` declaration per function of rt_b200.h, derived mechanically from the header (so the two
    cannot drift apart);
  * `impl Backend for B200Backend`: every method of the reference's trait (src/backend/mod.rs:14-656), each forwarding to
    one entry point, written from the tables below.

No Rust toolchain exists where this library is built, so the output is unverified source for a maintainer of the
reference; its compiled and tested twin is rusttensor_b200/csrc/host/b200_backend.hpp (same method list, same calls).

    python include/gen_rust_shim.py        # rewrites include/b200_backend.rs
"""
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))

C2RUST = {
    "rt_ctx*": "*mut RtCtx", "rt_ctx**": "*mut *mut RtCtx", "rt_graph*": "*mut RtGraph", "rt_graph**": "*mut *mut RtGraph",
    "rt_upload*": "*mut RtUpload", "rt_upload**": "*mut *mut RtUpload", "rt_event*": "*mut RtEvent", "rt_event**": "*mut *mut RtEvent",
    "int": "c_int", "int*": "*mut c_int", "const int*": "*const c_int", "int* const*": "*const *mut c_int",
    "int32_t": "i32", "const int32_t*": "*const i32", "int64_t": "i64", "int64_t*": "*mut i64", "const int64_t*": "*const i64",
    "uint32_t": "u32", "uint64_t": "u64", "uint64_t*": "*mut u64", "size_t": "usize", "float": "f32", "float*": "*mut f32", "const float*": "*const f32",
    "double*": "*mut f64", "float* const*": "*const *mut f32", "const float* const*": "*const *const f32",
    "void*": "*mut c_void", "void**": "*mut *mut c_void", "const void*": "*const c_void", "void* const*": "*const *mut c_void",
    "rt_upload* const*": "*const *mut RtUpload",
    "const uint8_t*": "*const u8", "uint8_t*": "*mut u8", "rt_status": "RtStatus", "const char*": "*const c_char", "void": "()",
}


def parse_header():
    text = open(os.path.join(HERE, "rt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = []
    for ret, name, args in re.findall(r"\b(rt_status|const char\*|int|void\*)\s+(rt_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        params = []
        for a in [x.strip() for x in " ".join(args.split()).split(",")]:
            if a in ("void", ""):
                continue
            m = re.match(r"(.*?)(\w+)(\[[A-Z_]+\])?$", a)
            ctype, pname, arr = m.group(1).strip(), m.group(2), m.group(3)
            ctype = re.sub(r"\s*\*\s*", "*", ctype).replace("*const*", "* const*")
            if arr:  # fixed-size byte arrays decay to pointers
                ctype = ctype + "*"
            if pname in ("type", "ref", "in", "move", "box"):
                pname += "_"
            params.append((pname, C2RUST[ctype]))
        out.append((name, params, C2RUST[ret]))
    return out


def ffi_block():
    lines = []
    for name, params, ret in parse_header():
        sig = ", ".join(f"{n}: {t}" for n, t in params)
        lines.append(f"        pub fn {name}({sig})" + (f" -> {ret};" if ret != "()" else ";"))
    return "\n".join(lines)


UNARY = [  # (trait method, enum constant)
    ("exp", "RT_EXP"), ("ln", "RT_LN"), ("relu", "RT_RELU"), ("sigmoid", "RT_SIGMOID"), ("abs", "RT_ABS"), ("sqrt", "RT_SQRT"),
    ("tanh", "RT_TANH"), ("softplus", "RT_SOFTPLUS"), ("square", "RT_SQUARE"), ("sin", "RT_SIN"), ("cos", "RT_COS"), ("tan", "RT_TAN")]
BINARY = [("mul", "RT_MUL"), ("add", "RT_ADD"), ("sub", "RT_SUB"), ("div", "RT_DIV"), ("powf", "RT_POWF"), ("maximum", "RT_MAXIMUM"),
          ("minimum", "RT_MINIMUM"), ("equal", "RT_EQUAL"), ("not_equal", "RT_NOT_EQUAL"), ("greater", "RT_GREATER"),
          ("greater_equal", "RT_GREATER_EQUAL"), ("less", "RT_LESS"), ("less_equal", "RT_LESS_EQUAL")]
BINARY_BWD = ["mul", "add", "sub", "div", "powf", "maximum", "minimum"]
REDUCE_OPT = [("max", "RT_RED_MAX"), ("min", "RT_RED_MIN"), ("prod", "RT_RED_PROD"), ("logsumexp", "RT_RED_LOGSUMEXP"), ("mean", "RT_RED_MEAN")]
REDUCE_BWD = [("max_backward", "RT_RED_MAX", "Max"), ("min_backward", "RT_RED_MIN", "Min"), ("prod_backward", "RT_RED_PROD", "Prod"),
              ("logsumexp_backward", "RT_RED_LOGSUMEXP", "LogSumExp"), ("mean_backward", "RT_RED_MEAN", "Mean"),
              ("sum_backward", "RT_RED_SUM", "Sum")]


def enum_consts():
    text = open(os.path.join(HERE, "rt_b200.h")).read()
    out, seen = [], set()
    for body in re.findall(r"enum\s*\{(.*?)\};", text, flags=re.S):
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        for name, val in re.findall(r"\b(RT_[A-Z0-9_]+)\s*=\s*(\d+)", body):
            if name not in seen:
                seen.add(name)
                out.append(f"    pub const {name}: c_int = {val};")
    return "\n".join(out)


def impl_block():
    m = []
    a = m.append
    for name, code in UNARY:
        a(f"    fn {name}(x: &Self::Storage) -> Result<Self::Storage, Error> {{ unary({code}, x, 0.0, 0.0) }}")
        a(f"    fn {name}_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {{ unary_bwd({code}, op, g, 0.0, 0.0) }}")
    for name, code in BINARY:
        a(f"    fn {name}(a: &Self::Storage, b: &Self::Storage) -> Result<Self::Storage, Error> {{ binary({code}, \"{name}\", a, b) }}")
    for name in BINARY_BWD:
        a(f"    fn {name}_backward(op: &Op<Self>, g: &Self::Storage) -> Result<(Self::Storage, Self::Storage), Error> {{ binary_bwd(RT_{name.upper()}, op, g) }}")
    for name, code in REDUCE_OPT:
        a(f"    fn {name}(x: &Self::Storage, axis: Option<usize>) -> Result<Self::Storage, Error> {{ reduce({code}, x, axis) }}")
    for name, code, variant in REDUCE_BWD:
        a(f"    fn {name}(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {{")
        a(f"        let axis = match op.op_type {{ OpType::{variant}(a) => a, _ => return Err(Error::InternalLogicError(\"{name}: wrong op type\".into())) }};")
        a(f"        reduce_bwd({code}, &*op.inputs[0].data(), g, axis)")
        a("    }")
    return "\n".join(m)


TEMPLATE = r'''// b200_backend.rs -- `impl Backend for B200Backend` over the C ABI of rt_b200.h.
//
// GENERATED by include/gen_rust_shim.py from include/rt_b200.h; do not edit by hand.
// UNVERIFIED SOURCE: no Rust toolchain exists where librt_b200.so is built.  It is what a maintainer of the reference would
// add as src/backend/b200/mod.rs (feature "b200"); the compiled and tested twin with the same method list and the same
// calls is rusttensor_b200/csrc/host/b200_backend.hpp.  Citations are lines of the reference's src/backend/mod.rs.
#![allow(clippy::too_many_arguments)]
use crate::backend::Backend;
use crate::error::Error;
use crate::graph::{Op, OpType};
use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_void};
use std::sync::{Arc, Mutex, OnceLock};

pub mod ffi {
    use super::*;
    #[repr(C)] pub struct RtCtx { _p: [u8; 0] }
    #[repr(C)] pub struct RtGraph { _p: [u8; 0] }
    #[repr(C)] pub struct RtUpload { _p: [u8; 0] }
    #[repr(C)] pub struct RtEvent { _p: [u8; 0] }
    pub type RtStatus = i32;
@ENUMS@
    #[link(name = "rt_b200")]
    extern "C" {
@FFI@
    }
}
use ffi::*;

// ---- context: one per process and device, like the reference's global CUDA context (src/backend/cuda/context.rs) ----
struct CtxPtr(*mut RtCtx);
unsafe impl Send for CtxPtr {}
unsafe impl Sync for CtxPtr {}
static CTX: OnceLock<CtxPtr> = OnceLock::new();
static RNG: Mutex<(u64, u64)> = Mutex::new((0x5eed, 0)); // (seed, counter offset) of the random factories
fn ctx() -> *mut RtCtx {
    CTX.get_or_init(|| {
        let mut c: *mut RtCtx = std::ptr::null_mut();
        let dev = std::env::var("LOCAL_RANK").ok().and_then(|s| s.parse().ok()).unwrap_or(0);
        let st = unsafe { rt_ctx_create(dev, &mut c) };
        assert_eq!(st, RT_OK, "rt_ctx_create failed: this backend needs a CUDA device (sm_100a)");
        CtxPtr(c)
    }).0
}

fn check(st: RtStatus) -> Result<(), Error> {
    if st == RT_OK { return Ok(()); }
    let msg = unsafe { CStr::from_ptr(rt_last_error(ctx())) }.to_string_lossy().into_owned();
    Err(match st {
        RT_ERR_SHAPE_MISMATCH => Error::ShapeMismatch { expected: vec![], actual: vec![] }, // shapes are checked host side first, with details
        RT_ERR_INCOMPATIBLE_SHAPES => Error::IncompatibleShapes { op: msg, shape_a: vec![], shape_b: vec![] },
        RT_ERR_INVALID_INDEX => Error::InvalidIndex(vec![]),
        RT_ERR_INVALID_OPERATION => Error::InvalidOperation(msg),
        RT_ERR_INTERNAL => Error::InternalLogicError(msg),
        RT_ERR_DIMENSION_MISMATCH => Error::DimensionMismatch(0, 0),
        RT_ERR_OOM => Error::OutOfMemory,
        RT_ERR_UNIMPLEMENTED => Error::Unimplemented(msg),
        RT_ERR_EMPTY_TENSOR => Error::EmptyTensor,
        RT_ERR_INITIALIZATION => Error::InitializationError,
        _ => Error::CudaError(msg), // RT_ERR_CUDA, RT_ERR_TIMEOUT, RT_ERR_NCCL
    })
}

// ---- storage: a reference-counted device buffer + shape.  Buffers are immutable once produced, so `Clone` (an Arc
// clone) is observably the deep copy the trait asks for (mod.rs:39); the in-place methods copy on write. ----
#[derive(Debug)]
struct DeviceBuf { ptr: *mut f32, bytes: usize }
unsafe impl Send for DeviceBuf {}
unsafe impl Sync for DeviceBuf {}
impl Drop for DeviceBuf { fn drop(&mut self) { if !self.ptr.is_null() { unsafe { rt_free(ctx(), self.ptr as *mut c_void) }; } } }

#[derive(Debug, Clone)]
pub struct B200Storage { buf: Arc<DeviceBuf>, shape: Vec<usize> }
impl std::fmt::Display for B200Storage {
    fn fmt(&self, f: &mut std::fmt::Formatter) -> std::fmt::Result { write!(f, "B200Storage{:?}", self.shape) }
}
impl B200Storage {
    fn alloc(shape: &[usize]) -> Result<Self, Error> {
        let n: usize = shape.iter().product();
        let mut p: *mut c_void = std::ptr::null_mut();
        check(unsafe { rt_malloc(ctx(), 4 * n.max(1), &mut p) })?;
        Ok(Self { buf: Arc::new(DeviceBuf { ptr: p as *mut f32, bytes: 4 * n.max(1) }), shape: shape.to_vec() })
    }
    fn ptr(&self) -> *const f32 { self.buf.ptr }
    fn ptr_mut(&self) -> *mut f32 { self.buf.ptr } // fresh outputs only
    fn numel(&self) -> usize { self.shape.iter().product() }
    fn dims(&self) -> Vec<i64> { self.shape.iter().map(|&d| d as i64).collect() }
    fn unique_ptr_mut(&mut self) -> Result<*mut f32, Error> { // copy on write before an in-place update
        if Arc::strong_count(&self.buf) > 1 {
            let c = Self::alloc(&self.shape)?;
            check(unsafe { rt_memcpy_d2d(ctx(), c.buf.ptr as *mut c_void, self.buf.ptr as *const c_void, 4 * self.numel()) })?;
            self.buf = c.buf;
        }
        Ok(self.buf.ptr)
    }
}

// [outer, len, inner] view of `shape` around `axis`
fn split(shape: &[usize], axis: usize) -> (i64, i64, i64) {
    (shape[..axis].iter().product::<usize>() as i64, shape[axis] as i64, shape[axis + 1..].iter().product::<usize>() as i64)
}
fn broadcast_shape(op: &str, a: &[usize], b: &[usize]) -> Result<Vec<usize>, Error> {
    crate::util::broadcast_shapes(a, b).map_err(|_| Error::IncompatibleShapes { op: op.into(), shape_a: a.to_vec(), shape_b: b.to_vec() })
}
fn unary(code: c_int, x: &B200Storage, p0: f32, p1: f32) -> Result<B200Storage, Error> {
    let out = B200Storage::alloc(&x.shape)?;
    check(unsafe { rt_unary(ctx(), code, x.ptr(), out.ptr_mut(), x.numel() as i64, p0, p1) })?;
    Ok(out)
}
fn unary_bwd(code: c_int, op: &Op<B200Backend>, g: &B200Storage, p0: f32, p1: f32) -> Result<B200Storage, Error> {
    let x = &*op.inputs[0].data(); // f' is recomputed from the INPUT, as in the reference's CPU backend
    if x.shape != g.shape { return Err(Error::ShapeMismatch { expected: x.shape.clone(), actual: g.shape.clone() }); }
    let out = B200Storage::alloc(&x.shape)?;
    check(unsafe { rt_unary_backward(ctx(), code, x.ptr(), g.ptr(), out.ptr_mut(), x.numel() as i64, p0, p1) })?;
    Ok(out)
}
fn binary(code: c_int, name: &str, a: &B200Storage, b: &B200Storage) -> Result<B200Storage, Error> {
    let out = B200Storage::alloc(&broadcast_shape(name, &a.shape, &b.shape)?)?;
    let (da, db) = (a.dims(), b.dims());
    check(unsafe { rt_binary(ctx(), code, a.ptr(), da.as_ptr(), da.len() as c_int, b.ptr(), db.as_ptr(), db.len() as c_int, out.ptr_mut()) })?;
    Ok(out)
}
fn binary_bwd(code: c_int, op: &Op<B200Backend>, g: &B200Storage) -> Result<(B200Storage, B200Storage), Error> {
    let (a, b) = (&*op.inputs[0].data(), &*op.inputs[1].data());
    let (ga, gb) = (B200Storage::alloc(&a.shape)?, B200Storage::alloc(&b.shape)?); // un-broadcast inside the kernels
    let (da, db) = (a.dims(), b.dims());
    check(unsafe { rt_binary_backward(ctx(), code, a.ptr(), da.as_ptr(), da.len() as c_int, b.ptr(), db.as_ptr(), db.len() as c_int,
                                      g.ptr(), ga.ptr_mut(), gb.ptr_mut()) })?;
    Ok((ga, gb))
}
fn reduce(kind: c_int, x: &B200Storage, axis: Option<usize>) -> Result<B200Storage, Error> {
    let (shape, (o, l, i)) = match axis {
        None => (vec![], (1, x.numel() as i64, 1)),           // global reductions have shape [] (mod.rs:293)
        Some(a) if a < x.shape.len() => { let mut s = x.shape.clone(); s.remove(a); (s, split(&x.shape, a)) }
        Some(a) => return Err(Error::InvalidIndex(vec![a])),
    };
    let out = B200Storage::alloc(&shape)?;
    check(unsafe { rt_reduce(ctx(), kind, x.ptr(), o, l, i, out.ptr_mut()) })?;
    Ok(out)
}
fn reduce_bwd(kind: c_int, x: &B200Storage, g: &B200Storage, axis: Option<usize>) -> Result<B200Storage, Error> {
    let (o, l, i) = match axis { None => (1, x.numel() as i64, 1), Some(a) => split(&x.shape, a) };
    let out = B200Storage::alloc(&x.shape)?;
    check(unsafe { rt_reduce_backward(ctx(), kind, x.ptr(), g.ptr(), o, l, i, out.ptr_mut()) })?;
    Ok(out)
}
fn random(shape: &[usize], f: impl Fn(*mut f32, i64, u64, u64) -> RtStatus) -> Result<B200Storage, Error> {
    let out = B200Storage::alloc(shape)?;
    let n = out.numel();
    if n == 0 { return B200Backend::zeros(shape); }
    let mut st = RNG.lock().unwrap();
    check(f(out.ptr_mut(), n as i64, st.0, st.1))?;
    st.1 += ((n + 3) / 4) as u64; // a call consumes (n + 3) / 4 counter values
    Ok(out)
}

#[derive(Debug, Clone, Copy)]
pub struct B200Backend;

impl Backend for B200Backend {
    type Storage = B200Storage;

    // ---- factories and access (mod.rs:44-88, 248-252) ----
    fn zeros(shape: &[usize]) -> Result<Self::Storage, Error> {
        let s = B200Storage::alloc(shape)?;
        check(unsafe { rt_fill(ctx(), s.ptr_mut(), 0.0, s.numel() as i64) })?;
        Ok(s)
    }
    fn ones(shape: &[usize]) -> Result<Self::Storage, Error> {
        let s = B200Storage::alloc(shape)?;
        check(unsafe { rt_fill(ctx(), s.ptr_mut(), 1.0, s.numel() as i64) })?;
        Ok(s)
    }
    fn from_vec(data: Vec<f32>, shape: &[usize]) -> Result<Self::Storage, Error> {
        let n: usize = shape.iter().product();
        if data.len() != n { return Err(Error::ShapeMismatch { expected: shape.to_vec(), actual: vec![data.len()] }); }
        let s = B200Storage::alloc(shape)?;
        check(unsafe { rt_memcpy_h2d(ctx(), s.ptr_mut() as *mut c_void, data.as_ptr() as *const c_void, 4 * n) })?;
        Ok(s)
    }
    fn kaiming_uniform(fan_in: usize, shape: &[usize]) -> Result<Self::Storage, Error> {            // mod.rs:57, src/init.rs:7-52
        if shape.is_empty() { return Err(Error::InvalidOperation("Cannot initialize tensor with empty shape".into())); }
        if shape.iter().any(|&d| d == 0) { return Self::zeros(shape); }
        if fan_in == 0 { return Err(Error::InvalidOperation("Fan-in cannot be zero for Kaiming initialization".into())); }
        let bound = (6.0 / fan_in as f32).sqrt();
        Self::random_uniform(shape, -bound, bound)
    }
    fn random_uniform(shape: &[usize], low: f32, high: f32) -> Result<Self::Storage, Error> {        // mod.rs:63
        random(shape, |p, n, seed, off| unsafe { rt_random_uniform(ctx(), p, n, low, high, seed, off) })
    }
    fn random_normal(shape: &[usize], mean: f32, std_dev: f32) -> Result<Self::Storage, Error> {     // mod.rs:66
        random(shape, |p, n, seed, off| unsafe { rt_random_normal(ctx(), p, n, mean, std_dev, seed, off) })
    }
    fn bernoulli(shape: &[usize], p: f32) -> Result<Self::Storage, Error> {                          // mod.rs:69
        random(shape, |q, n, seed, off| unsafe { rt_bernoulli(ctx(), q, n, p, seed, off) })
    }
    fn device(_s: &Self::Storage) -> crate::Device { crate::Device::Cuda(0) }
    fn shape(s: &Self::Storage) -> &[usize] { &s.shape }
    fn size(s: &Self::Storage) -> usize { s.numel() }
    fn into_raw_vec(s: Self::Storage) -> Result<Vec<f32>, Error> { Self::copy_to_host(&s) }
    fn set_data(s: &mut Self::Storage, data: Self::Storage) -> Result<(), Error> { *s = data; Ok(()) }
    fn set_shape(s: &mut Self::Storage, shape: &[usize]) -> Result<(), Error> {
        if shape.iter().product::<usize>() != s.numel() { return Err(Error::ShapeMismatch { expected: shape.to_vec(), actual: s.shape.clone() }); }
        s.shape = shape.to_vec();
        Ok(())
    }
    fn copy_to_host(s: &Self::Storage) -> Result<Vec<f32>, Error> {                                  // mod.rs:248 (synchronises)
        let mut v = vec![0f32; s.numel()];
        check(unsafe { rt_memcpy_d2h(ctx(), v.as_mut_ptr() as *mut c_void, s.ptr() as *const c_void, 4 * v.len()) })?;
        Ok(v)
    }
    fn update_from_host(s: &mut Self::Storage, data: &[f32]) -> Result<(), Error> {                  // mod.rs:252
        if data.len() != s.numel() { return Err(Error::ShapeMismatch { expected: s.shape.clone(), actual: vec![data.len()] }); }
        let p = s.unique_ptr_mut()?;
        check(unsafe { rt_memcpy_h2d(ctx(), p as *mut c_void, data.as_ptr() as *const c_void, 4 * data.len()) })
    }
    fn map<F>(x: &Self::Storage, f: F) -> Result<Self::Storage, Error> where F: Fn(f32) -> f32 + Send + Sync + 'static {
        let v: Vec<f32> = Self::copy_to_host(x)?.into_iter().map(f).collect(); // an arbitrary host closure: host round trip, as in the reference's CUDA backend
        Self::from_vec(v, &x.shape)
    }

    // ---- element-wise, comparisons, reductions and their gradients (one forwarding call each) ----
@IMPL@
    fn elu(x: &Self::Storage, alpha: f32) -> Result<Self::Storage, Error> { unary(RT_ELU, x, alpha, 0.0) }
    fn elu_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {
        let alpha = match op.op_type { OpType::Elu(a) => a, _ => return Err(Error::InternalLogicError("elu_backward: wrong op type".into())) };
        unary_bwd(RT_ELU, op, g, alpha, 0.0)
    }
    fn clip(x: &Self::Storage, min_val: f32, max_val: f32) -> Result<Self::Storage, Error> { unary(RT_CLIP, x, min_val, max_val) }
    fn clip_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {
        let (lo, hi) = match op.op_type { OpType::Clip { min_val, max_val } => (min_val, max_val), _ => return Err(Error::InternalLogicError("clip_backward: wrong op type".into())) };
        unary_bwd(RT_CLIP, op, g, lo, hi)
    }
    fn mul_scalar(x: &Self::Storage, scalar: f32) -> Result<Self::Storage, Error> { unary(RT_MUL_SCALAR, x, scalar, 0.0) }
    fn div_scalar(x: &Self::Storage, scalar: f32) -> Result<Self::Storage, Error> {
        if scalar == 0.0 { return Err(Error::InvalidOperation("Division by zero scalar".into())); }
        unary(RT_DIV_SCALAR, x, scalar, 0.0)
    }
    fn sum_along_axis(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> { reduce(RT_RED_SUM, x, Some(axis)) }
    fn max_along_axis(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> { reduce(RT_RED_MAX, x, Some(axis)) }
    fn argmax(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> { reduce(RT_RED_ARGMAX, x, Some(axis)) }
    fn argmin(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> { reduce(RT_RED_ARGMIN, x, Some(axis)) }
    fn sum_all(x: &Self::Storage) -> Result<f32, Error> {                                            // mod.rs:293 (synchronises)
        let mut v = 0f32;
        check(unsafe { rt_sum_all_host(ctx(), x.ptr(), x.numel() as i64, &mut v) })?;
        Ok(v)
    }
    fn log_softmax(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> {                 // mod.rs:307
        let (o, l, i) = split(&x.shape, axis);
        let out = B200Storage::alloc(&x.shape)?;
        check(unsafe { rt_log_softmax(ctx(), x.ptr(), o, l, i, out.ptr_mut()) })?;
        Ok(out)
    }
    fn log_softmax_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {      // mod.rs:349
        let axis = match op.op_type { OpType::LogSoftmax(a) => a, _ => return Err(Error::InternalLogicError("log_softmax_backward: wrong op type".into())) };
        let x = &*op.inputs[0].data();
        let (o, l, i) = split(&x.shape, axis);
        let out = B200Storage::alloc(&x.shape)?;
        check(unsafe { rt_log_softmax_backward(ctx(), x.ptr(), g.ptr(), o, l, i, out.ptr_mut()) })?;
        Ok(out)
    }

    // ---- layout ----
    fn transpose(x: &Self::Storage) -> Result<Self::Storage, Error> {                                // mod.rs:275 (matrices)
        if x.shape.len() != 2 { return Err(Error::Unimplemented("transpose of tensors with more than two axes".into())); }
        let out = B200Storage::alloc(&[x.shape[1], x.shape[0]])?;
        check(unsafe { rt_transpose2d(ctx(), x.ptr(), x.shape[0] as i64, x.shape[1] as i64, out.ptr_mut()) })?;
        Ok(out)
    }
    fn broadcast_to(x: &Self::Storage, shape: &[usize]) -> Result<Self::Storage, Error> {            // mod.rs:277
        let out = B200Storage::alloc(shape)?;
        let (dx, ds): (Vec<i64>, Vec<i64>) = (x.dims(), shape.iter().map(|&d| d as i64).collect());
        check(unsafe { rt_broadcast_to(ctx(), x.ptr(), dx.as_ptr(), dx.len() as c_int, ds.as_ptr(), ds.len() as c_int, out.ptr_mut()) })?;
        Ok(out)
    }
    fn slice(x: &Self::Storage, ranges: &[std::ops::Range<usize>]) -> Result<Self::Storage, Error> { // mod.rs:522
        let shape: Vec<usize> = ranges.iter().map(|r| r.end - r.start).collect();
        let out = B200Storage::alloc(&shape)?;
        let (dx, st, os): (Vec<i64>, Vec<i64>, Vec<i64>) = (x.dims(), ranges.iter().map(|r| r.start as i64).collect(), shape.iter().map(|&d| d as i64).collect());
        check(unsafe { rt_slice(ctx(), x.ptr(), dx.as_ptr(), dx.len() as c_int, st.as_ptr(), os.as_ptr(), out.ptr_mut()) })?;
        Ok(out)
    }
    fn slice_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {            // mod.rs:535: zero fill + write the block
        let (input_shape, ranges) = match &op.op_type { OpType::Slice { input_shape, ranges } => (input_shape, ranges), _ => return Err(Error::InternalLogicError("slice_backward: wrong op type".into())) };
        let out = Self::zeros(input_shape)?;
        let (ds, st, gs): (Vec<i64>, Vec<i64>, Vec<i64>) = (out.dims(), ranges.iter().map(|r| r.start as i64).collect(), g.dims());
        check(unsafe { rt_slice_assign(ctx(), out.ptr_mut(), ds.as_ptr(), ds.len() as c_int, st.as_ptr(), g.ptr(), gs.as_ptr()) })?;
        Ok(out)
    }
    fn concat(tensors: &[&Self::Storage], axis: usize) -> Result<Self::Storage, Error> {            // mod.rs:550: one block write per input
        let mut shape = tensors[0].shape.clone();
        shape[axis] = tensors.iter().map(|t| t.shape[axis]).sum();
        let out = B200Storage::alloc(&shape)?;
        let ds = out.dims();
        let mut start = vec![0i64; shape.len()];
        for t in tensors {
            let ts = t.dims();
            check(unsafe { rt_slice_assign(ctx(), out.ptr_mut(), ds.as_ptr(), ds.len() as c_int, start.as_ptr(), t.ptr(), ts.as_ptr()) })?;
            start[axis] += t.shape[axis] as i64;
        }
        Ok(out)
    }
    fn concat_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Vec<Self::Storage>, Error> {      // mod.rs:563: one slice per input
        let (axis, shapes) = match &op.op_type { OpType::Concat { axis, input_shapes } => (*axis, input_shapes), _ => return Err(Error::InternalLogicError("concat_backward: wrong op type".into())) };
        let mut start = 0usize;
        let mut outs = Vec::with_capacity(shapes.len());
        for s in shapes {
            let ranges: Vec<std::ops::Range<usize>> = s.iter().enumerate().map(|(d, &n)| if d == axis { start..start + n } else { 0..n }).collect();
            outs.push(Self::slice(g, &ranges)?);
            start += s[axis];
        }
        Ok(outs)
    }
    fn expand_dims(x: &Self::Storage, axis: usize) -> Result<Self::Storage, Error> {                 // metadata only: the buffer is shared
        let mut s = x.clone();
        s.shape.insert(axis, 1);
        Ok(s)
    }
    fn expand_dims_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {
        let mut s = g.clone();
        s.shape = op.inputs[0].data().shape.clone();
        Ok(s)
    }
    fn squeeze(x: &Self::Storage, axis: Option<usize>) -> Result<Self::Storage, Error> {
        let mut s = x.clone();
        match axis {
            Some(a) => { if s.shape.get(a) != Some(&1) { return Err(Error::InvalidOperation("squeeze: axis extent is not 1".into())); } s.shape.remove(a); }
            None => s.shape.retain(|&d| d != 1),
        }
        Ok(s)
    }
    fn squeeze_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {
        let shape = match &op.op_type { OpType::Squeeze { original_input_shape, .. } => original_input_shape.clone(), _ => return Err(Error::InternalLogicError("squeeze_backward: wrong op type".into())) };
        let mut s = g.clone();
        s.shape = shape;
        Ok(s)
    }

    // ---- contractions ----
    fn matmul(a: &Self::Storage, b: &Self::Storage) -> Result<Self::Storage, Error> {                // mod.rs:93
        if a.shape.len() != 2 || b.shape.len() != 2 || a.shape[1] != b.shape[0] {
            return Err(Error::IncompatibleShapes { op: "matmul".into(), shape_a: a.shape.clone(), shape_b: b.shape.clone() });
        }
        let (m, k, n) = (a.shape[0] as i64, a.shape[1] as i64, b.shape[1] as i64);
        let out = B200Storage::alloc(&[m as usize, n as usize])?;
        check(unsafe { rt_gemm(ctx(), 0, 0, m, n, k, a.ptr(), k, b.ptr(), n, out.ptr_mut(), n, 0) })?;
        Ok(out)
    }
    fn matmul_backward(op: &Op<Self>, g: &Self::Storage) -> Result<(Self::Storage, Self::Storage), Error> { // mod.rs:324: g*B^T, A^T*g, no transposes materialised
        let (a, b) = (&*op.inputs[0].data(), &*op.inputs[1].data());
        let (da, db) = (B200Storage::alloc(&a.shape)?, B200Storage::alloc(&b.shape)?);
        check(unsafe { rt_matmul_backward(ctx(), a.ptr(), b.ptr(), g.ptr(), a.shape[0] as i64, a.shape[1] as i64, b.shape[1] as i64, da.ptr_mut(), db.ptr_mut()) })?;
        Ok((da, db))
    }
    fn conv2d(x: &Self::Storage, w: &Self::Storage, bias: Option<&Self::Storage>, stride: (usize, usize), padding: (usize, usize)) -> Result<Self::Storage, Error> { // mod.rs:101
        let (n, cin, h, wd, cout, kh, kw) = (x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], w.shape[2], w.shape[3]);
        let (ho, wo) = ((h + 2 * padding.0 - kh) / stride.0 + 1, (wd + 2 * padding.1 - kw) / stride.1 + 1);
        let out = B200Storage::alloc(&[n, cout, ho, wo])?;
        check(unsafe { rt_conv2d(ctx(), x.ptr(), w.ptr(), bias.map_or(std::ptr::null(), |b| b.ptr()), n as i64, cin as i64, h as i64, wd as i64, cout as i64,
                                 kh as c_int, kw as c_int, stride.0 as c_int, stride.1 as c_int, padding.0 as c_int, padding.1 as c_int, out.ptr_mut()) })?;
        Ok(out)
    }
    fn conv2d_backward(x: &Self::Storage, w: &Self::Storage, g: &Self::Storage, stride: (usize, usize), padding: (usize, usize))
        -> Result<(Self::Storage, Self::Storage, Option<Self::Storage>), Error> {                      // mod.rs:111
        let (dx, dw, db) = (B200Storage::alloc(&x.shape)?, B200Storage::alloc(&w.shape)?, B200Storage::alloc(&[w.shape[0]])?);
        check(unsafe { rt_conv2d_backward(ctx(), x.ptr(), w.ptr(), g.ptr(), x.shape[0] as i64, x.shape[1] as i64, x.shape[2] as i64, x.shape[3] as i64,
                                          w.shape[0] as i64, w.shape[2] as c_int, w.shape[3] as c_int, stride.0 as c_int, stride.1 as c_int,
                                          padding.0 as c_int, padding.1 as c_int, dx.ptr_mut(), dw.ptr_mut(), db.ptr_mut()) })?;
        Ok((dx, dw, Some(db)))
    }
    fn conv2d_transpose(x: &Self::Storage, w: &Self::Storage, bias: Option<&Self::Storage>, stride: (usize, usize), padding: (usize, usize)) -> Result<Self::Storage, Error> { // mod.rs:125
        let (n, cin, h, wd, cout, kh, kw) = (x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[1], w.shape[2], w.shape[3]);
        let (oh, ow) = ((h - 1) * stride.0 + kh - 2 * padding.0, (wd - 1) * stride.1 + kw - 2 * padding.1);
        let out = B200Storage::alloc(&[n, cout, oh, ow])?;
        check(unsafe { rt_conv2d_transpose(ctx(), x.ptr(), w.ptr(), bias.map_or(std::ptr::null(), |b| b.ptr()), n as i64, cin as i64, h as i64, wd as i64, cout as i64,
                                           kh as c_int, kw as c_int, stride.0 as c_int, stride.1 as c_int, padding.0 as c_int, padding.1 as c_int, out.ptr_mut()) })?;
        Ok(out)
    }
    fn conv2d_transpose_backward(x: &Self::Storage, w: &Self::Storage, g: &Self::Storage, stride: (usize, usize), padding: (usize, usize))
        -> Result<(Self::Storage, Self::Storage, Option<Self::Storage>), Error> {                      // mod.rs:135
        let (dx, dw, db) = (B200Storage::alloc(&x.shape)?, B200Storage::alloc(&w.shape)?, B200Storage::alloc(&[w.shape[1]])?);
        check(unsafe { rt_conv2d_transpose_backward(ctx(), x.ptr(), w.ptr(), g.ptr(), x.shape[0] as i64, x.shape[1] as i64, x.shape[2] as i64, x.shape[3] as i64,
                                                    w.shape[1] as i64, w.shape[2] as c_int, w.shape[3] as c_int, stride.0 as c_int, stride.1 as c_int,
                                                    padding.0 as c_int, padding.1 as c_int, dx.ptr_mut(), dw.ptr_mut(), db.ptr_mut()) })?;
        Ok((dx, dw, Some(db)))
    }
    fn max_pool2d(x: &Self::Storage, kernel_size: (usize, usize), stride: (usize, usize), padding: (usize, usize)) -> Result<(Self::Storage, Self::Storage), Error> { // mod.rs:144
        let (n, c, h, w) = (x.shape[0], x.shape[1], x.shape[2], x.shape[3]);
        let (ho, wo) = ((h + 2 * padding.0 - kernel_size.0) / stride.0 + 1, (w + 2 * padding.1 - kernel_size.1) / stride.1 + 1);
        let (y, idx) = (B200Storage::alloc(&[n, c, ho, wo])?, B200Storage::alloc(&[n, c, ho, wo])?);
        check(unsafe { rt_max_pool2d(ctx(), x.ptr(), n as i64, c as i64, h as i64, w as i64, kernel_size.0 as c_int, kernel_size.1 as c_int,
                                     stride.0 as c_int, stride.1 as c_int, padding.0 as c_int, padding.1 as c_int, y.ptr_mut(), idx.ptr_mut()) })?;
        Ok((y, idx))
    }
    fn max_pool2d_backward(op: &Op<Self>, g: &Self::Storage) -> Result<Self::Storage, Error> {       // mod.rs:151: inputs = [x, indices]
        let (k, s, p) = match op.op_type { OpType::MaxPool2D { kernel_size, stride, padding } => (kernel_size, stride, padding), _ => return Err(Error::InternalLogicError("max_pool2d_backward: wrong op type".into())) };
        let (x, idx) = (&*op.inputs[0].data(), &*op.inputs[1].data());
        let dx = B200Storage::alloc(&x.shape)?;
        check(unsafe { rt_max_pool2d_backward(ctx(), g.ptr(), idx.ptr(), x.shape[0] as i64, x.shape[1] as i64, x.shape[2] as i64, x.shape[3] as i64,
                                              k.0 as c_int, k.1 as c_int, s.0 as c_int, s.1 as c_int, p.0 as c_int, p.1 as c_int, dx.ptr_mut()) })?;
        Ok(dx)
    }

    // ---- optimizer steps, in place (mod.rs:18-36, 256-272) ----
    fn sgd_step(w: &mut Self::Storage, dw: &Self::Storage, lr: f32) -> Result<(), Error> {
        let n = w.numel() as i64;
        check(unsafe { rt_sgd_step(ctx(), w.unique_ptr_mut()?, dw.ptr(), n, lr) })
    }
    fn momentum_sgd_step(p: &mut Self::Storage, g: &Self::Storage, v: &mut Self::Storage, lr: f32, momentum: f32) -> Result<(), Error> {
        let n = p.numel() as i64;
        check(unsafe { rt_momentum_sgd_step(ctx(), p.unique_ptr_mut()?, g.ptr(), v.unique_ptr_mut()?, n, lr, momentum) })
    }
    fn adagrad_step(p: &mut Self::Storage, g: &Self::Storage, acc: &mut Self::Storage, lr: f32, epsilon: f32) -> Result<(), Error> {
        let n = p.numel() as i64;
        check(unsafe { rt_adagrad_step(ctx(), p.unique_ptr_mut()?, g.ptr(), acc.unique_ptr_mut()?, n, lr, epsilon) })
    }
    fn adam_step(p: &mut Self::Storage, g: &Self::Storage, m: &mut Self::Storage, v: &mut Self::Storage, lr: f32, beta1: f32, beta2: f32,
                 epsilon: f32, t: usize) -> Result<(), Error> {
        let n = p.numel() as i64;
        check(unsafe { rt_adam_step(ctx(), p.unique_ptr_mut()?, g.ptr(), m.unique_ptr_mut()?, v.unique_ptr_mut()?, n, lr, beta1, beta2, epsilon, t as i64) })
    }
}
'''


def main():
    out = TEMPLATE.replace("@ENUMS@", enum_consts()).replace("@FFI@", ffi_block()).replace("@IMPL@", impl_block())
    path = os.path.join(HERE, "b200_backend.rs")
    with open(path, "w") as f:
        f.write(out)
    print(f"wrote {path}: {len(parse_header())} extern functions")


if __name__ == "__main__":
    main()
