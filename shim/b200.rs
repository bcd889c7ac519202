//! `impl Backend for B200Backend`: catgrad's interpreter backend trait over the C ABI of libcatgrad_b200.so
//! (include/catgrad_b200.h).
//!
//! Where it goes: `catgrad/src/interpreter/backend/b200.rs`, behind a cargo feature `b200-backend`
//! (`pub mod b200;` next to `pub mod ndarray;` / `pub mod candle;` in backend/mod.rs), with
//! `println!("cargo:rustc-link-lib=dylib=catgrad_b200")` and the library's directory as a
//! `cargo:rustc-link-search` in the crate's build script.  Nothing above the trait changes: `Interpreter<B>`,
//! `tensor_op()`, the typechecker and every model definition are generic in `B: Backend`.
//!
//! This file is shipped as source: the image this library is built in has no Rust toolchain, so it has not been
//! compiled.  Every method is the same three steps (unwrap the handles of the tagged tuple, call the entry point of
//! the same name, re-tag the result with the dtype the library reports), written once in `call*` helpers.
//!
//! Error behaviour mirrors the existing backends: trait methods are infallible by type, so a non-zero status
//! panics with the library's message (for a shape mismatch that message starts with "Shape mismatch in
//! operation", the text the candle backend panics with); the `ndarray_from_vec_*` constructors return
//! `BackendError::ShapeError` for status 8.

use super::{Backend, BackendError, BackendTensorOps};
use crate::category::core::{Dtype, Shape};
use crate::interpreter::types::*;
use float8::F8E4M3;
use half::{bf16, f16};
use std::ffi::{c_char, c_int, c_void, CStr};
use std::sync::Arc;

#[repr(C)]
pub struct CgCtx {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct CgTensor {
    _opaque: [u8; 0],
}

type Unary = unsafe extern "C" fn(*mut CgCtx, *const CgTensor, *mut *mut CgTensor) -> c_int;
type Binary = unsafe extern "C" fn(*mut CgCtx, *const CgTensor, *const CgTensor, *mut *mut CgTensor) -> c_int;

extern "C" {
    fn cg_init(device: c_int, out: *mut *mut CgCtx) -> c_int;
    fn cg_destroy(ctx: *mut CgCtx);
    fn cg_last_error(ctx: *mut CgCtx) -> *const c_char;
    fn cg_release(t: *mut CgTensor);
    fn cg_rank(t: *const CgTensor) -> c_int;
    fn cg_shape(t: *const CgTensor, dims: *mut u64, rank: *mut c_int) -> c_int;
    fn cg_dtype_of(t: *const CgTensor) -> c_int;

    fn cg_zeros(ctx: *mut CgCtx, dims: *const u64, rank: c_int, dtype: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_from_vec_f32(ctx: *mut CgCtx, data: *const f32, n: u64, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_from_vec_f16(ctx: *mut CgCtx, data: *const u16, n: u64, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_from_vec_bf16(ctx: *mut CgCtx, data: *const u16, n: u64, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_from_vec_fp8(ctx: *mut CgCtx, data: *const u8, n: u64, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_from_vec_u32(ctx: *mut CgCtx, data: *const u32, n: u64, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_arange(ctx: *mut CgCtx, end: u64, out: *mut *mut CgTensor) -> c_int;

    fn cg_cast(ctx: *mut CgCtx, x: *const CgTensor, dtype: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_matmul(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_add(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_sub(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_mul(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_div(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_pow(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_lt(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_gt(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_gte(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_lte(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_eq(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_where_cond(ctx: *mut CgCtx, mask: *const CgTensor, x: *const CgTensor, y: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_sin(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_cos(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_exp(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_log(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_floor(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_round(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_neg(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_broadcast(ctx: *mut CgCtx, x: *const CgTensor, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_reshape(ctx: *mut CgCtx, x: *const CgTensor, dims: *const u64, rank: c_int, out: *mut *mut CgTensor) -> c_int;
    fn cg_transpose(ctx: *mut CgCtx, x: *const CgTensor, d0: u64, d1: u64, out: *mut *mut CgTensor) -> c_int;
    fn cg_max(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_sum(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_argmax(ctx: *mut CgCtx, x: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_topk(ctx: *mut CgCtx, x: *const CgTensor, k: u64, values: *mut *mut CgTensor, indices: *mut *mut CgTensor) -> c_int;
    fn cg_compare(ctx: *mut CgCtx, a: *const CgTensor, b: *const CgTensor, equal: *mut c_int) -> c_int;
    fn cg_concat(ctx: *mut CgCtx, x: *const CgTensor, y: *const CgTensor, dim: u64, out: *mut *mut CgTensor) -> c_int;
    fn cg_index(ctx: *mut CgCtx, x: *const CgTensor, dim: u64, indices: *const CgTensor, out: *mut *mut CgTensor) -> c_int;
    fn cg_slice(ctx: *mut CgCtx, x: *const CgTensor, dim: u64, start: u64, len: u64, out: *mut *mut CgTensor) -> c_int;
    fn cg_to_bool(ctx: *mut CgCtx, x: *const CgTensor, out: *mut c_int) -> c_int;
    fn cg_to_vec(ctx: *mut CgCtx, x: *const CgTensor, dst: *mut c_void, cap_bytes: u64) -> c_int;
    fn cg_format(ctx: *mut CgCtx, x: *const CgTensor, buf: *mut c_char, cap: u64) -> c_int;
}

/// One device + one stream.  `Interpreter` is single-threaded (the engine above it is `Rc`-based), so the context is
/// only ever entered from one thread at a time; the `Send + Sync` the trait asks of tensors is for moving values.
#[derive(Debug)]
struct CtxHandle(*mut CgCtx);
unsafe impl Send for CtxHandle {}
unsafe impl Sync for CtxHandle {}
impl Drop for CtxHandle {
    fn drop(&mut self) {
        unsafe { cg_destroy(self.0) }
    }
}

/// Owning tensor handle; releasing is thread-safe in the library.
#[derive(Debug)]
pub struct Handle {
    raw: *mut CgTensor,
    _ctx: Arc<CtxHandle>, // keeps the context alive as long as any tensor
}
unsafe impl Send for Handle {}
unsafe impl Sync for Handle {}
impl Drop for Handle {
    fn drop(&mut self) {
        unsafe { cg_release(self.raw) }
    }
}

/// `Copy` edges of a term clone the value (eval.rs `apply_copy`): cloning the Arc shares the device buffer.
#[derive(Clone, Debug)]
pub struct B200Tensor(Arc<Handle>);

impl BackendTensorOps for B200Tensor {
    fn shape(&self) -> Shape {
        let mut dims = [0u64; 8];
        let mut rank: c_int = 0;
        unsafe { cg_shape(self.0.raw, dims.as_mut_ptr(), &mut rank) };
        Shape(dims[..rank as usize].iter().map(|&d| d as usize).collect())
    }
}

#[derive(Clone, Debug)]
pub struct B200Backend {
    ctx: Arc<CtxHandle>,
}

fn dtype_code(d: &Dtype) -> c_int {
    match d {
        Dtype::F32 => 0,
        Dtype::F16 => 1,
        Dtype::BF16 => 2,
        Dtype::F8 => 3,
        Dtype::U32 => 4,
    }
}

fn dims_of(shape: &Shape) -> Vec<u64> {
    shape.0.iter().map(|&d| d as u64).collect()
}

impl B200Backend {
    /// Fails (instead of falling back to a CPU path) when the device is not a B200 or the library cannot start.
    pub fn new(device: i32) -> Result<Self, String> {
        let mut raw: *mut CgCtx = std::ptr::null_mut();
        let st = unsafe { cg_init(device as c_int, &mut raw) };
        if st != 0 || raw.is_null() {
            let msg = unsafe { CStr::from_ptr(cg_last_error(std::ptr::null_mut())) };
            return Err(format!("cg_init({device}): status {st}: {}", msg.to_string_lossy()));
        }
        Ok(Self { ctx: Arc::new(CtxHandle(raw)) })
    }

    fn message(&self) -> String {
        unsafe { CStr::from_ptr(cg_last_error(self.ctx.0)) }.to_string_lossy().into_owned()
    }

    fn check(&self, status: c_int) {
        if status != 0 {
            panic!("{}", self.message());
        }
    }

    fn wrap(&self, raw: *mut CgTensor) -> B200Tensor {
        B200Tensor(Arc::new(Handle { raw, _ctx: self.ctx.clone() }))
    }

    /// Re-tags a fresh handle with the dtype the library reports for it.
    fn tag(&self, raw: *mut CgTensor) -> TaggedTensor<Self> {
        let t = self.wrap(raw);
        match unsafe { cg_dtype_of(raw) } {
            0 => TaggedTensor::F32([t]),
            1 => TaggedTensor::F16([t]),
            2 => TaggedTensor::BF16([t]),
            3 => TaggedTensor::FP8([t]),
            _ => TaggedTensor::U32([t]),
        }
    }

    fn one(x: &TaggedTensor<Self>) -> *const CgTensor {
        match x {
            TaggedTensor::F32([a]) | TaggedTensor::F16([a]) | TaggedTensor::BF16([a]) | TaggedTensor::FP8([a])
            | TaggedTensor::U32([a]) => a.0.raw,
        }
    }

    fn two(x: &TaggedTensorTuple<Self, 2>) -> (*const CgTensor, *const CgTensor) {
        match x {
            TaggedTensorTuple::F32([a, b]) | TaggedTensorTuple::F16([a, b]) | TaggedTensorTuple::BF16([a, b])
            | TaggedTensorTuple::FP8([a, b]) | TaggedTensorTuple::U32([a, b]) => (a.0.raw, b.0.raw),
        }
    }

    fn call1(&self, f: Unary, x: TaggedTensor<Self>) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { f(self.ctx.0, Self::one(&x), &mut out) });
        self.tag(out)
    }

    fn call2(&self, f: Binary, args: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> {
        let (a, b) = Self::two(&args);
        let mut out = std::ptr::null_mut();
        self.check(unsafe { f(self.ctx.0, a, b, &mut out) });
        self.tag(out)
    }

    fn from_vec<T>(
        &self,
        f: unsafe extern "C" fn(*mut CgCtx, *const T, u64, *const u64, c_int, *mut *mut CgTensor) -> c_int,
        data: *const T,
        n: usize,
        shape: Shape,
    ) -> Result<TaggedTensor<Self>, BackendError> {
        let dims = dims_of(&shape);
        let mut out = std::ptr::null_mut();
        match unsafe { f(self.ctx.0, data, n as u64, dims.as_ptr(), dims.len() as c_int, &mut out) } {
            0 => Ok(self.tag(out)),
            8 => Err(BackendError::ShapeError),
            _ => panic!("{}", self.message()),
        }
    }
}

impl Backend for B200Backend {
    type BackendTensor = B200Tensor;

    fn zeros(&self, shape: Shape, target_dtype: Dtype) -> TaggedTensor<Self> {
        let dims = dims_of(&shape);
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_zeros(self.ctx.0, dims.as_ptr(), dims.len() as c_int, dtype_code(&target_dtype), &mut out) });
        self.tag(out)
    }

    fn ndarray_from_vec_f32(&self, data: Vec<f32>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        self.from_vec(cg_from_vec_f32, data.as_ptr(), data.len(), shape)
    }
    // half::f16, half::bf16 and float8::F8E4M3 are transparent wrappers of their bit patterns
    fn ndarray_from_vec_f16(&self, data: Vec<f16>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        self.from_vec(cg_from_vec_f16, data.as_ptr() as *const u16, data.len(), shape)
    }
    fn ndarray_from_vec_bf16(&self, data: Vec<bf16>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        self.from_vec(cg_from_vec_bf16, data.as_ptr() as *const u16, data.len(), shape)
    }
    fn ndarray_from_vec_fp8(&self, data: Vec<F8E4M3>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        self.from_vec(cg_from_vec_fp8, data.as_ptr() as *const u8, data.len(), shape)
    }
    fn ndarray_from_vec_u32(&self, data: Vec<u32>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        self.from_vec(cg_from_vec_u32, data.as_ptr(), data.len(), shape)
    }

    fn cast(&self, x: TaggedTensor<Self>, target_dtype: Dtype) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_cast(self.ctx.0, Self::one(&x), dtype_code(&target_dtype), &mut out) });
        self.tag(out)
    }

    fn matmul(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_matmul, lhs) }
    fn add(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_add, lhs) }
    fn sub(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_sub, lhs) }
    fn mul(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_mul, lhs) }
    fn div(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_div, lhs) }
    fn pow(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_pow, lhs) }
    fn lt(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_lt, lhs) }
    fn gt(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_gt, lhs) }
    fn gte(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_gte, lhs) }
    fn lte(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_lte, lhs) }
    fn eq(&self, lhs: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.call2(cg_eq, lhs) }

    fn where_cond(&self, args: TaggedTensorTuple<Self, 3>) -> TaggedTensor<Self> {
        let (m, x, y) = match &args {
            TaggedTensorTuple::F32([m, x, y]) | TaggedTensorTuple::F16([m, x, y]) | TaggedTensorTuple::BF16([m, x, y])
            | TaggedTensorTuple::FP8([m, x, y]) | TaggedTensorTuple::U32([m, x, y]) => (m.0.raw, x.0.raw, y.0.raw),
        };
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_where_cond(self.ctx.0, m, x, y, &mut out) });
        self.tag(out)
    }

    fn sin(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_sin, x) }
    fn cos(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_cos, x) }
    fn exp(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_exp, x) }
    fn log(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_log, x) }
    fn floor(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_floor, x) }
    fn round(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_round, x) }
    fn neg(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_neg, x) }
    fn max(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_max, x) }
    fn sum(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_sum, x) }
    fn argmax(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.call1(cg_argmax, x) }

    fn broadcast(&self, x: TaggedTensor<Self>, shape: Shape) -> TaggedTensor<Self> {
        let dims = dims_of(&shape);
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_broadcast(self.ctx.0, Self::one(&x), dims.as_ptr(), dims.len() as c_int, &mut out) });
        self.tag(out)
    }
    fn reshape(&self, x: TaggedTensor<Self>, new_shape: Shape) -> TaggedTensor<Self> {
        let dims = dims_of(&new_shape);
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_reshape(self.ctx.0, Self::one(&x), dims.as_ptr(), dims.len() as c_int, &mut out) });
        self.tag(out)
    }
    fn transpose(&self, x: TaggedTensor<Self>, dim0: usize, dim1: usize) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_transpose(self.ctx.0, Self::one(&x), dim0 as u64, dim1 as u64, &mut out) });
        self.tag(out)
    }

    fn topk(&self, x: TaggedTensor<Self>, k: usize) -> (TaggedTensor<Self>, TaggedTensor<Self>) {
        let (mut v, mut i) = (std::ptr::null_mut(), std::ptr::null_mut());
        self.check(unsafe { cg_topk(self.ctx.0, Self::one(&x), k as u64, &mut v, &mut i) });
        (self.tag(v), self.tag(i))
    }

    fn compare(&self, x: TaggedTensorTuple<Self, 2>) -> bool {
        let (a, b) = Self::two(&x);
        let mut eq: c_int = 0;
        self.check(unsafe { cg_compare(self.ctx.0, a, b, &mut eq) });
        eq != 0
    }

    fn concat(&self, x: TaggedTensor<Self>, y: TaggedTensor<Self>, dim: usize) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_concat(self.ctx.0, Self::one(&x), Self::one(&y), dim as u64, &mut out) });
        self.tag(out)
    }
    fn index(&self, x: TaggedTensor<Self>, dim: usize, indices: TaggedTensor<Self>) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_index(self.ctx.0, Self::one(&x), dim as u64, Self::one(&indices), &mut out) });
        self.tag(out)
    }
    fn slice(&self, x: TaggedTensor<Self>, dim: usize, start: usize, len: usize) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_slice(self.ctx.0, Self::one(&x), dim as u64, start as u64, len as u64, &mut out) });
        self.tag(out)
    }
    fn arange(&self, end: usize) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { cg_arange(self.ctx.0, end as u64, &mut out) });
        self.tag(out)
    }

    fn to_bool(&self, x: TaggedTensor<Self>) -> bool {
        let mut b: c_int = 0;
        self.check(unsafe { cg_to_bool(self.ctx.0, Self::one(&x), &mut b) });
        b != 0
    }

    /// Synchronises the stream (one of the four calls that do) and copies the elements out in logical order.
    fn to_vec(&self, vec: TaggedTensor<Self>) -> TaggedVec {
        let n: usize = vec.shape().0.iter().product();
        let raw = Self::one(&vec);
        macro_rules! read {
            ($t:ty, $variant:ident) => {{
                let mut v: Vec<$t> = Vec::with_capacity(n);
                self.check(unsafe { cg_to_vec(self.ctx.0, raw, v.as_mut_ptr() as *mut c_void, (n * std::mem::size_of::<$t>()) as u64) });
                unsafe { v.set_len(n) };
                TaggedVec::$variant(v)
            }};
        }
        match vec {
            TaggedTensor::F32(_) => read!(f32, F32),
            TaggedTensor::F16(_) => read!(f16, F16),
            TaggedTensor::BF16(_) => read!(bf16, BF16),
            TaggedTensor::FP8(_) => read!(F8E4M3, FP8),
            TaggedTensor::U32(_) => read!(u32, U32),
        }
    }

    fn format_tensor(&self, tensor: &TaggedTensor<Self>) -> String {
        let mut buf = vec![0 as c_char; 1 << 16];
        self.check(unsafe { cg_format(self.ctx.0, Self::one(tensor), buf.as_mut_ptr(), buf.len() as u64) });
        unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
    }
}
