/*
 * oracle.h — CPU restatement of the catgrad `NdArrayBackend`
 * (catgrad/src/interpreter/backend/ndarray.rs) behind the same C ABI shape as
 * include/catgrad_cuda.h, with the prefix `cgo_`.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the parity checker and the timed CPU
 * baseline.  Nothing in the product package may load it; only tests/, the smoke entry
 * and the benchmark's cpu-baseline / reference arm do.
 *
 * Parity pin: the reference is Rust and cannot be compiled in this environment (no rustc,
 * no vendored crates), so the oracle is pinned against every golden vector the reference's
 * own tests hold at this boundary (ndarray.rs:630-821, catgrad/tests/test_interpreter.rs:
 * 85-226, and the legacy known-answer tests for the same formulas,
 * catgrad-llm/src/legacy/nn/layers.rs:735-1563).  Whole-model logits and greedy tokens are
 * fixed by no reference test: that part is "parity unpinned".
 *
 * Arithmetic that lives in third-party crates absent from the reference tree:
 *   ndarray 0.17.1        sum_axis / fold_axis / select / broadcast / to_shape / concatenate
 *   matrixmultiply 0.3.10 f32 GEMM (accumulation order not reproducible here)
 *   Rust std f32::{powf,sin,cos} -> the platform libm, which this file calls as well.
 */
#ifndef CATGRAD_ORACLE_H
#define CATGRAD_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct cgo_ctx cgo_ctx;
typedef struct cgo_tensor cgo_tensor;

/* `threads` <= 0 means all host cores.  The reference's ndarray build is single-threaded
 * (catgrad/Cargo.toml:17 enables neither rayon nor blas); more threads only make the
 * baseline faster than the reference could be. */
int32_t cgo_ctx_create(int32_t threads, cgo_ctx** out);
int32_t cgo_ctx_destroy(cgo_ctx* ctx);
const char* cgo_last_error(cgo_ctx* ctx);
int32_t cgo_ctx_threads(cgo_ctx* ctx);

int32_t cgo_tensor_retain(cgo_tensor* t);
int32_t cgo_tensor_release(cgo_tensor* t);
int32_t cgo_shape(const cgo_tensor* t, int32_t* rank, int64_t dims[8]);
int32_t cgo_dtype_of(const cgo_tensor* t, int32_t* dtype);

int32_t cgo_zeros(cgo_ctx*, const int64_t* dims, int32_t rank, int32_t dtype, cgo_tensor** out);
int32_t cgo_ndarray_from_vec_f32(cgo_ctx*, const float* data, int64_t n, const int64_t* dims, int32_t rank, cgo_tensor** out);
int32_t cgo_ndarray_from_vec_u32(cgo_ctx*, const uint32_t* data, int64_t n, const int64_t* dims, int32_t rank, cgo_tensor** out);
int32_t cgo_cast(cgo_ctx*, const cgo_tensor* x, int32_t dtype, cgo_tensor** out);
int32_t cgo_matmul(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_add(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_sub(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_mul(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_div(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_pow(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_lt(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_eq(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out);
int32_t cgo_sin(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_cos(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_neg(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_broadcast(cgo_ctx*, const cgo_tensor* x, const int64_t* dims, int32_t rank, cgo_tensor** out);
int32_t cgo_reshape(cgo_ctx*, const cgo_tensor* x, const int64_t* dims, int32_t rank, cgo_tensor** out);
int32_t cgo_transpose(cgo_ctx*, const cgo_tensor* x, int32_t dim0, int32_t dim1, cgo_tensor** out);
int32_t cgo_max(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_sum(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_argmax(cgo_ctx*, const cgo_tensor* x, cgo_tensor** out);
int32_t cgo_topk(cgo_ctx*, const cgo_tensor* x, int64_t k, cgo_tensor** values, cgo_tensor** indices);
int32_t cgo_compare(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, int32_t* equal);
int32_t cgo_concat(cgo_ctx*, const cgo_tensor* a, const cgo_tensor* b, int32_t dim, cgo_tensor** out);
int32_t cgo_index(cgo_ctx*, const cgo_tensor* x, int32_t dim, const cgo_tensor* indices, cgo_tensor** out);
int32_t cgo_slice(cgo_ctx*, const cgo_tensor* x, int32_t dim, int64_t start, int64_t len, cgo_tensor** out);
int32_t cgo_arange(cgo_ctx*, int64_t end, cgo_tensor** out);
int32_t cgo_to_vec_f32(cgo_ctx*, const cgo_tensor* x, float* dst, int64_t n);
int32_t cgo_to_vec_u32(cgo_ctx*, const cgo_tensor* x, uint32_t* dst, int64_t n);

#ifdef __cplusplus
}
#endif
#endif
