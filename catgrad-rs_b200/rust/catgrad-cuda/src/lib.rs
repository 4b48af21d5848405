// NOT compiled in this repository's build environment (no Rust toolchain): source only.
//
// `impl Backend for CudaBackend`: the catgrad interpreter trait
// (catgrad/src/interpreter/backend/mod.rs:22-82) over libcatgrad_cuda.so.  Usage is what the
// reference's example driver already does (catgrad-llm/examples/llama/main.rs:116):
//
//     let backend = catgrad_cuda::CudaBackend::new(0, Precision::BF16);
//     let interpreter = Interpreter::new(backend, stdlib(), parameter_values);
//
// Tensors are moved into trait methods and dropped there (cg_tensor_release); `Clone` is
// cg_tensor_retain (O(1)), which is what `apply_copy` (abstract_interpreter/eval.rs:104-113)
// relies on.  A non-zero status panics with the library's message, like the existing backends
// (ndarray.rs:212,255,293,333; candle.rs:413-415).
mod ffi;
pub mod decoder;

use catgrad::category::core::{Dtype, Shape};
use catgrad::interpreter::backend::{Backend, BackendError, BackendTensorOps};
use catgrad::interpreter::{TaggedTensor, TaggedTensorTuple, TaggedVec};
use std::ffi::CStr;
use std::sync::Arc;

#[derive(Clone, Copy, Debug)]
pub enum Precision { F32, BF16 }

struct Ctx(*mut ffi::cg_ctx);
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}
impl Drop for Ctx { fn drop(&mut self) { unsafe { ffi::cg_ctx_destroy(self.0); } } }

#[derive(Clone)]
pub struct CudaBackend { ctx: Arc<Ctx> }
impl std::fmt::Debug for CudaBackend {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "CudaBackend") }
}

/// One reference to a device tensor.
pub struct CudaTensor(*mut ffi::cg_tensor);
unsafe impl Send for CudaTensor {}
unsafe impl Sync for CudaTensor {}
impl Clone for CudaTensor {
    fn clone(&self) -> Self { unsafe { ffi::cg_tensor_retain(self.0); } CudaTensor(self.0) }
}
impl CudaTensor {
    pub(crate) fn raw(&self) -> *const ffi::cg_tensor { self.0 }
    /// Takes over one reference returned by the library.
    pub(crate) fn from_raw(p: *mut ffi::cg_tensor) -> Self { CudaTensor(p) }
}
impl Drop for CudaTensor { fn drop(&mut self) { unsafe { ffi::cg_tensor_release(self.0); } } }
impl std::fmt::Debug for CudaTensor {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "CudaTensor{:?}", self.shape()) }
}
impl BackendTensorOps for CudaTensor {
    fn shape(&self) -> Shape {  // host metadata, no synchronisation
        let (mut rank, mut dims) = (0i32, [0i64; 8]);
        unsafe { ffi::cg_shape(self.0, &mut rank, dims.as_mut_ptr()); }
        Shape(dims[..rank as usize].iter().map(|&d| d as usize).collect())
    }
}

fn dims_of(s: &Shape) -> Vec<i64> { s.0.iter().map(|&d| d as i64).collect() }

impl CudaBackend {
    pub fn new(device: i32, precision: Precision) -> Self {
        let mut ctx = std::ptr::null_mut();
        let p = match precision { Precision::F32 => ffi::CG_PREC_F32, Precision::BF16 => ffi::CG_PREC_BF16 };
        let st = unsafe { ffi::cg_ctx_create(device, p, std::ptr::null_mut(), &mut ctx) };
        assert_eq!(st, 0, "cg_ctx_create failed: no CUDA device? (there is no CPU fallback)");
        CudaBackend { ctx: Arc::new(Ctx(ctx)) }
    }
    /// Record the trait calls instead of running them and fuse the stdlib's chains (rmsnorm, softmax,
    /// silu * up, rope, the attention core) when a result is needed.  The interpreter and the model
    /// graphs above stay exactly as they are.
    pub fn lazy(self, on: bool) -> Self {
        let name = std::ffi::CString::new("lazy").unwrap();
        self.check(unsafe { ffi::cg_set_option(self.ctx.0, name.as_ptr(), on as i64) });
        self
    }
    /// (trait calls recorded, chains fused, calls pending)
    pub fn lazy_stats(&self) -> (i64, i64, i64) {
        let (mut a, mut b, mut c) = (0i64, 0i64, 0i64);
        self.check(unsafe { ffi::cg_lazy_stats(self.ctx.0, &mut a, &mut b, &mut c) });
        (a, b, c)
    }
    /// y = x W^T for a weight stored [out, in] (tensor cores when W is stored bf16): what
    /// `linear_no_bias` lowers to, without the transposed view.
    pub fn linear(&self, x: &CudaTensor, w: &CudaTensor) -> CudaTensor {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { ffi::cg_linear(self.ctx.0, x.raw(), w.raw(), &mut out) });
        CudaTensor::from_raw(out)
    }
    /// act(x Wg^T) * (x Wu^T) for the stacked weight [2F, in] (gate rows first); act 0 = silu, 1 = tanh gelu.
    pub fn linear_glu(&self, x: &CudaTensor, w_gate_up: &CudaTensor, act: i32) -> CudaTensor {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { ffi::cg_linear_glu(self.ctx.0, x.raw(), w_gate_up.raw(), act, &mut out) });
        CudaTensor::from_raw(out)
    }
    /// Run everything pending and surface device-side errors.
    pub fn sync(&self) { self.check(unsafe { ffi::cg_sync(self.ctx.0) }); }
    pub(crate) fn raw_ctx(&self) -> *mut ffi::cg_ctx { self.ctx.0 }
    pub(crate) fn check(&self, st: i32) {
        if st != 0 {
            let msg = unsafe { CStr::from_ptr(ffi::cg_last_error(self.ctx.0)) }.to_string_lossy().into_owned();
            panic!("{msg}");
        }
    }
    fn un(&self, f: unsafe extern "C" fn(*mut ffi::cg_ctx, *const ffi::cg_tensor, *mut *mut ffi::cg_tensor) -> i32,
          x: &CudaTensor) -> CudaTensor {
        let mut out = std::ptr::null_mut();
        self.check(unsafe { f(self.ctx.0, x.0, &mut out) });
        CudaTensor(out)
    }
    fn bin(&self, f: unsafe extern "C" fn(*mut ffi::cg_ctx, *const ffi::cg_tensor, *const ffi::cg_tensor, *mut *mut ffi::cg_tensor) -> i32,
           args: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> {
        let mut out = std::ptr::null_mut();
        match args {
            TaggedTensorTuple::F32([a, b]) => { self.check(unsafe { f(self.ctx.0, a.0, b.0, &mut out) }); TaggedTensor::F32([CudaTensor(out)]) }
            TaggedTensorTuple::U32([a, b]) => { self.check(unsafe { f(self.ctx.0, a.0, b.0, &mut out) }); TaggedTensor::U32([CudaTensor(out)]) }
        }
    }
    fn map1(&self, x: TaggedTensor<Self>, g: impl Fn(&CudaTensor) -> CudaTensor) -> TaggedTensor<Self> {
        match x {
            TaggedTensor::F32([a]) => TaggedTensor::F32([g(&a)]),
            TaggedTensor::U32([a]) => TaggedTensor::U32([g(&a)]),
        }
    }
}

impl Backend for CudaBackend {
    type BackendTensor = CudaTensor;

    fn to_vec(&self, v: TaggedTensor<Self>) -> TaggedVec {
        match v {
            TaggedTensor::F32([x]) => {
                let n: usize = x.shape().0.iter().product();
                let mut out = vec![0f32; n];
                self.check(unsafe { ffi::cg_to_vec_f32(self.ctx.0, x.0, out.as_mut_ptr(), n as i64) });
                TaggedVec::F32(out)
            }
            TaggedTensor::U32([x]) => {
                let n: usize = x.shape().0.iter().product();
                let mut out = vec![0u32; n];
                self.check(unsafe { ffi::cg_to_vec_u32(self.ctx.0, x.0, out.as_mut_ptr(), n as i64) });
                TaggedVec::U32(out)
            }
        }
    }
    fn zeros(&self, shape: Shape, dtype: Dtype) -> TaggedTensor<Self> {
        let (d, mut out) = (dims_of(&shape), std::ptr::null_mut());
        let tag = if dtype == Dtype::F32 { ffi::CG_F32 } else { ffi::CG_U32 };
        self.check(unsafe { ffi::cg_zeros(self.ctx.0, d.as_ptr(), d.len() as i32, tag, &mut out) });
        if dtype == Dtype::F32 { TaggedTensor::F32([CudaTensor(out)]) } else { TaggedTensor::U32([CudaTensor(out)]) }
    }
    fn ndarray_from_vec_f32(&self, data: Vec<f32>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        let (d, mut out) = (dims_of(&shape), std::ptr::null_mut());
        let st = unsafe { ffi::cg_ndarray_from_vec_f32(self.ctx.0, data.as_ptr(), data.len() as i64, d.as_ptr(), d.len() as i32, &mut out) };
        if st == 1 { return Err(BackendError::ShapeError); }
        self.check(st);
        Ok(TaggedTensor::F32([CudaTensor(out)]))
    }
    fn ndarray_from_vec_u32(&self, data: Vec<u32>, shape: Shape) -> Result<TaggedTensor<Self>, BackendError> {
        let (d, mut out) = (dims_of(&shape), std::ptr::null_mut());
        let st = unsafe { ffi::cg_ndarray_from_vec_u32(self.ctx.0, data.as_ptr(), data.len() as i64, d.as_ptr(), d.len() as i32, &mut out) };
        if st == 1 { return Err(BackendError::ShapeError); }
        self.check(st);
        Ok(TaggedTensor::U32([CudaTensor(out)]))
    }
    fn cast(&self, x: TaggedTensor<Self>, dtype: Dtype) -> TaggedTensor<Self> {
        let tag = if dtype == Dtype::F32 { ffi::CG_F32 } else { ffi::CG_U32 };
        let t = match &x { TaggedTensor::F32([a]) | TaggedTensor::U32([a]) => a.clone() };
        let mut out = std::ptr::null_mut();
        self.check(unsafe { ffi::cg_cast(self.ctx.0, t.0, tag, &mut out) });
        if dtype == Dtype::F32 { TaggedTensor::F32([CudaTensor(out)]) } else { TaggedTensor::U32([CudaTensor(out)]) }
    }
    fn matmul(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_matmul, a) }
    fn add(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_add, a) }
    fn sub(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_sub, a) }
    fn mul(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_mul, a) }
    fn div(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_div, a) }
    fn pow(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_pow, a) }
    fn lt(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_lt, a) }
    fn eq(&self, a: TaggedTensorTuple<Self, 2>) -> TaggedTensor<Self> { self.bin(ffi::cg_eq, a) }
    fn sin(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.map1(x, |t| self.un(ffi::cg_sin, t)) }
    fn cos(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.map1(x, |t| self.un(ffi::cg_cos, t)) }
    fn neg(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.map1(x, |t| self.un(ffi::cg_neg, t)) }
    fn max(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.map1(x, |t| self.un(ffi::cg_max, t)) }
    fn sum(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> { self.map1(x, |t| self.un(ffi::cg_sum, t)) }
    fn argmax(&self, x: TaggedTensor<Self>) -> TaggedTensor<Self> {
        let t = match &x { TaggedTensor::F32([a]) | TaggedTensor::U32([a]) => a.clone() };
        TaggedTensor::U32([self.un(ffi::cg_argmax, &t)])
    }
    fn topk(&self, x: TaggedTensor<Self>, k: usize) -> (TaggedTensor<Self>, TaggedTensor<Self>) {
        let TaggedTensor::F32([t]) = x else { panic!("Unsupported type for topk") };
        let (mut v, mut i) = (std::ptr::null_mut(), std::ptr::null_mut());
        self.check(unsafe { ffi::cg_topk(self.ctx.0, t.0, k as i64, &mut v, &mut i) });
        (TaggedTensor::F32([CudaTensor(v)]), TaggedTensor::U32([CudaTensor(i)]))
    }
    fn broadcast(&self, x: TaggedTensor<Self>, shape: Shape) -> TaggedTensor<Self> {
        let d = dims_of(&shape);
        self.map1(x, |t| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_broadcast(self.ctx.0, t.0, d.as_ptr(), d.len() as i32, &mut o) }); CudaTensor(o) })
    }
    fn reshape(&self, x: TaggedTensor<Self>, shape: Shape) -> TaggedTensor<Self> {
        let d = dims_of(&shape);
        self.map1(x, |t| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_reshape(self.ctx.0, t.0, d.as_ptr(), d.len() as i32, &mut o) }); CudaTensor(o) })
    }
    fn transpose(&self, x: TaggedTensor<Self>, d0: usize, d1: usize) -> TaggedTensor<Self> {
        self.map1(x, |t| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_transpose(self.ctx.0, t.0, d0 as i32, d1 as i32, &mut o) }); CudaTensor(o) })
    }
    fn compare(&self, x: TaggedTensorTuple<Self, 2>) -> bool {
        let (a, b) = match &x { TaggedTensorTuple::F32([a, b]) | TaggedTensorTuple::U32([a, b]) => (a, b) };
        let mut eq = 0i32;
        self.check(unsafe { ffi::cg_compare(self.ctx.0, a.0, b.0, &mut eq) });
        eq != 0
    }
    fn concat(&self, x: TaggedTensor<Self>, y: TaggedTensor<Self>, dim: usize) -> TaggedTensor<Self> {
        let cat = |a: &CudaTensor, b: &CudaTensor| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_concat(self.ctx.0, a.0, b.0, dim as i32, &mut o) }); CudaTensor(o) };
        match (x, y) {
            (TaggedTensor::F32([a]), TaggedTensor::F32([b])) => TaggedTensor::F32([cat(&a, &b)]),
            (TaggedTensor::U32([a]), TaggedTensor::U32([b])) => TaggedTensor::U32([cat(&a, &b)]),
            _ => panic!("Incompatible types for concatenation"),
        }
    }
    fn index(&self, x: TaggedTensor<Self>, dim: usize, indices: TaggedTensor<Self>) -> TaggedTensor<Self> {
        let TaggedTensor::U32([ix]) = indices else { panic!("Invalid input types for indexing") };
        self.map1(x, |t| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_index(self.ctx.0, t.0, dim as i32, ix.0, &mut o) }); CudaTensor(o) })
    }
    fn slice(&self, x: TaggedTensor<Self>, dim: usize, start: usize, len: usize) -> TaggedTensor<Self> {
        self.map1(x, |t| { let mut o = std::ptr::null_mut(); self.check(unsafe { ffi::cg_slice(self.ctx.0, t.0, dim as i32, start as i64, len as i64, &mut o) }); CudaTensor(o) })
    }
    fn arange(&self, end: usize) -> TaggedTensor<Self> {
        let mut o = std::ptr::null_mut();
        self.check(unsafe { ffi::cg_arange(self.ctx.0, end as i64, &mut o) });
        TaggedTensor::U32([CudaTensor(o)])
    }
}
