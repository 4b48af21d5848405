// NOT compiled in this repository's build environment (no Rust toolchain): source only.
// Raw bindings to include/catgrad_cuda.h (trait-level subset + decoder runner).
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_void};

#[repr(C)] pub struct cg_ctx { _p: [u8; 0] }
#[repr(C)] pub struct cg_tensor { _p: [u8; 0] }

pub const CG_F32: i32 = 0;
pub const CG_U32: i32 = 1;
pub const CG_PREC_F32: i32 = 0;
pub const CG_PREC_BF16: i32 = 1;

type T = *mut cg_tensor;
type C = *mut cg_ctx;

extern "C" {
    pub fn cg_ctx_create(device: i32, precision: i32, stream: *mut c_void, out: *mut C) -> i32;
    pub fn cg_ctx_destroy(ctx: C) -> i32;
    pub fn cg_last_error(ctx: C) -> *const c_char;
    pub fn cg_tensor_retain(t: T) -> i32;
    pub fn cg_tensor_release(t: T) -> i32;
    pub fn cg_shape(t: *const cg_tensor, rank: *mut i32, dims: *mut i64) -> i32;
    pub fn cg_zeros(ctx: C, dims: *const i64, rank: i32, dtype: i32, out: *mut T) -> i32;
    pub fn cg_ndarray_from_vec_f32(ctx: C, data: *const f32, n: i64, dims: *const i64, rank: i32, out: *mut T) -> i32;
    pub fn cg_ndarray_from_vec_u32(ctx: C, data: *const u32, n: i64, dims: *const i64, rank: i32, out: *mut T) -> i32;
    pub fn cg_cast(ctx: C, x: *const cg_tensor, dtype: i32, out: *mut T) -> i32;
    pub fn cg_matmul(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_add(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_sub(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_mul(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_div(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_pow(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_lt(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_eq(ctx: C, a: *const cg_tensor, b: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_sin(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_cos(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_neg(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_broadcast(ctx: C, x: *const cg_tensor, dims: *const i64, rank: i32, out: *mut T) -> i32;
    pub fn cg_reshape(ctx: C, x: *const cg_tensor, dims: *const i64, rank: i32, out: *mut T) -> i32;
    pub fn cg_transpose(ctx: C, x: *const cg_tensor, d0: i32, d1: i32, out: *mut T) -> i32;
    pub fn cg_max(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_sum(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_argmax(ctx: C, x: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_topk(ctx: C, x: *const cg_tensor, k: i64, values: *mut T, indices: *mut T) -> i32;
    pub fn cg_compare(ctx: C, a: *const cg_tensor, b: *const cg_tensor, equal: *mut i32) -> i32;
    pub fn cg_concat(ctx: C, a: *const cg_tensor, b: *const cg_tensor, dim: i32, out: *mut T) -> i32;
    pub fn cg_index(ctx: C, x: *const cg_tensor, dim: i32, idx: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_slice(ctx: C, x: *const cg_tensor, dim: i32, start: i64, len: i64, out: *mut T) -> i32;
    pub fn cg_arange(ctx: C, end: i64, out: *mut T) -> i32;
    pub fn cg_to_vec_f32(ctx: C, x: *const cg_tensor, dst: *mut f32, n: i64) -> i32;
    pub fn cg_to_vec_u32(ctx: C, x: *const cg_tensor, dst: *mut u32, n: i64) -> i32;
    // extensions the shim exposes
    pub fn cg_sync(ctx: C) -> i32;
    pub fn cg_set_option(ctx: C, name: *const c_char, value: i64) -> i32;
    pub fn cg_lazy_stats(ctx: C, recorded: *mut i64, fused: *mut i64, pending: *mut i64) -> i32;
    pub fn cg_linear(ctx: C, x: *const cg_tensor, w: *const cg_tensor, out: *mut T) -> i32;
    pub fn cg_linear_glu(ctx: C, x: *const cg_tensor, w: *const cg_tensor, act: i32, out: *mut T) -> i32;
}
