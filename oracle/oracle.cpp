// oracle.cpp — CPU restatement of catgrad's NdArrayBackend.  TEST INFRASTRUCTURE ONLY:
// the parity checker and the timed CPU baseline; the product never loads it.
//
// Every function cites the reference lines it follows
// (catgrad/src/interpreter/backend/ndarray.rs unless another file is named).
// Parity pin and the third-party arithmetic this cannot reproduce are stated in oracle.h.
//
// Like the reference, every op returns a freshly materialised array in standard
// (row-major, contiguous) layout, except `transpose`, which copies and then swaps two
// axes so its result is non-contiguous (ndarray.rs:363-371).

#include "oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <numeric>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

namespace {

enum { ST_OK = 0, ST_SHAPE = 1, ST_DTYPE = 2, ST_INVALID = 3, ST_OOM = 5, ST_INDEX = 6 };
enum { DT_F32 = 0, DT_U32 = 1 };

struct Buf {
  uint32_t* p = nullptr;
  explicit Buf(int64_t n) {
    size_t bytes = (size_t)std::max<int64_t>(n, 1) * 4;
    bytes = (bytes + 63) / 64 * 64;
    p = (uint32_t*)aligned_alloc(64, bytes);
  }
  ~Buf() { free(p); }
};

}  // namespace

struct cgo_ctx {
  int threads = 1;
  std::string err;
};

struct cgo_tensor {
  std::atomic<int> rc{1};
  int dtype = DT_F32;
  std::vector<int64_t> shape, strides;  // strides in elements
  std::shared_ptr<Buf> buf;
  int64_t offset = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
  bool contiguous() const {
    int64_t s = 1;
    for (int i = (int)shape.size() - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != s) return false;
      s *= shape[i];
    }
    return true;
  }
  const uint32_t* raw() const { return buf->p + offset; }
  uint32_t* raw() { return buf->p + offset; }
};

namespace {

int fail(cgo_ctx* c, int code, const char* msg) {
  if (c) c->err = msg;
  return code;
}

std::vector<int64_t> row_major(const std::vector<int64_t>& shape) {
  std::vector<int64_t> st(shape.size());
  int64_t s = 1;
  for (int i = (int)shape.size() - 1; i >= 0; --i) {
    st[i] = s;
    s *= shape[i];
  }
  return st;
}

cgo_tensor* fresh(int dtype, const std::vector<int64_t>& shape) {
  auto* t = new cgo_tensor();
  t->dtype = dtype;
  t->shape = shape;
  t->strides = row_major(shape);
  t->buf = std::make_shared<Buf>(t->numel());
  return t;
}

// Gather a strided array into row-major order (what `to_owned()` / `to_shape()` do to a
// non-standard layout in the reference).
void gather(const cgo_tensor* t, uint32_t* dst) {
  const int64_t n = t->numel();
  if (n == 0) return;
  if (t->contiguous()) {
    memcpy(dst, t->raw(), (size_t)n * 4);
    return;
  }
  const int r = (int)t->shape.size();
  const int64_t inner = t->shape[r - 1], istr = t->strides[r - 1];
  const int64_t outer = n / inner;
  const uint32_t* src = t->raw();
#pragma omp parallel for schedule(static) if (n > (1 << 16))
  for (int64_t o = 0; o < outer; ++o) {
    int64_t rem = o, off = 0;
    for (int d = r - 2; d >= 0; --d) {
      off += (rem % t->shape[d]) * t->strides[d];
      rem /= t->shape[d];
    }
    uint32_t* out = dst + o * inner;
    const uint32_t* in = src + off;
    if (istr == 1) memcpy(out, in, (size_t)inner * 4);
    else for (int64_t i = 0; i < inner; ++i) out[i] = in[i * istr];
  }
}

// Pointer to row-major data of t; copies into `hold` when t is strided.
const uint32_t* contig(const cgo_tensor* t, std::unique_ptr<Buf>& hold) {
  if (t->contiguous()) return t->raw();
  hold.reset(new Buf(t->numel()));
  gather(t, hold->p);
  return hold->p;
}

inline float asf(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
inline uint32_t asu(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

// Rust `f32 as u32`: saturating, NaN -> 0 (ndarray.rs:99-104).
inline uint32_t f32_as_u32(float v) {
  if (!(v == v)) return 0u;
  if (v <= 0.0f) return 0u;
  if (v >= 4294967296.0f) return 0xFFFFFFFFu;
  return (uint32_t)v;
}

// Key that orders f32 bit patterns like Rust's f32::total_cmp.
inline uint32_t total_key(uint32_t bits) {
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// u32::pow with release-mode wrapping (ndarray.rs:449-453).
inline uint32_t pow_u32(uint32_t a, uint32_t b) {
  uint32_t r = 1;
  while (b) {
    if (b & 1) r *= a;
    a *= a;
    b >>= 1;
  }
  return r;
}

// Sum of a contiguous lane the way ndarray's eight-lane unrolled fold orders it
// (third-party: ndarray 0.17.1 numeric_util, reached from sum_axis at ndarray.rs:528).
template <class T>
T lane_sum(const T* xs, int64_t n) {
  T p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; ++j) p[j] = p[j] + xs[i + j];
  T acc = 0;
  acc = acc + (p[0] + p[4]);
  acc = acc + (p[1] + p[5]);
  acc = acc + (p[2] + p[6]);
  acc = acc + (p[3] + p[7]);
  for (; i < n; ++i) acc = acc + xs[i];
  return acc;
}

// ------------------------------------------------------------------ f32 GEMM ----------
// Stands in for matrixmultiply 0.3.10 (third-party, absent).  C[M,N] = A[M,K] B[K,N], all
// row-major.  Packed-panel blocking, 6x16 AVX2/FMA micro-kernel, K accumulated in order
// inside a 256-deep block and block after block.
constexpr int MR = 6, NR = 16, KC = 256, NC = 4096;

#if defined(__AVX2__) && defined(__FMA__)
inline void micro_6x16(int kc, const float* ap, const float* bp, float* c, int64_t ldc, bool add,
                       int mr, int nr) {
  __m256 acc[MR][2];
  for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm256_setzero_ps();
  for (int k = 0; k < kc; ++k) {
    __m256 b0 = _mm256_load_ps(bp + k * NR), b1 = _mm256_load_ps(bp + k * NR + 8);
    for (int i = 0; i < MR; ++i) {
      __m256 a = _mm256_broadcast_ss(ap + k * MR + i);
      acc[i][0] = _mm256_fmadd_ps(a, b0, acc[i][0]);
      acc[i][1] = _mm256_fmadd_ps(a, b1, acc[i][1]);
    }
  }
  if (mr == MR && nr == NR) {
    for (int i = 0; i < MR; ++i) {
      float* row = c + i * ldc;
      if (add) {
        _mm256_storeu_ps(row, _mm256_add_ps(_mm256_loadu_ps(row), acc[i][0]));
        _mm256_storeu_ps(row + 8, _mm256_add_ps(_mm256_loadu_ps(row + 8), acc[i][1]));
      } else {
        _mm256_storeu_ps(row, acc[i][0]);
        _mm256_storeu_ps(row + 8, acc[i][1]);
      }
    }
  } else {
    alignas(32) float tmp[MR][NR];
    for (int i = 0; i < MR; ++i) {
      _mm256_store_ps(tmp[i], acc[i][0]);
      _mm256_store_ps(tmp[i] + 8, acc[i][1]);
    }
    for (int i = 0; i < mr; ++i)
      for (int j = 0; j < nr; ++j) c[i * ldc + j] = add ? c[i * ldc + j] + tmp[i][j] : tmp[i][j];
  }
}
#else
inline void micro_6x16(int kc, const float* ap, const float* bp, float* c, int64_t ldc, bool add,
                       int mr, int nr) {
  float acc[MR][NR] = {};
  for (int k = 0; k < kc; ++k)
    for (int i = 0; i < MR; ++i)
      for (int j = 0; j < NR; ++j) acc[i][j] = fmaf(ap[k * MR + i], bp[k * NR + j], acc[i][j]);
  for (int i = 0; i < mr; ++i)
    for (int j = 0; j < nr; ++j) c[i * ldc + j] = add ? c[i * ldc + j] + acc[i][j] : acc[i][j];
}
#endif

void sgemm(int64_t M, int64_t N, int64_t K, const float* A, const float* B, float* C) {
  if (M == 0 || N == 0) return;
  if (K == 0) {
    memset(C, 0, (size_t)(M * N) * 4);
    return;
  }
  const int64_t mpanels = (M + MR - 1) / MR;
  std::unique_ptr<Buf> apack(new Buf(mpanels * MR * KC));
  std::unique_ptr<Buf> bpack(new Buf((int64_t)((std::min<int64_t>(N, NC) + NR - 1) / NR) * NR * KC));
  float* Ap = (float*)apack->p;
  float* Bp = (float*)bpack->p;
  for (int64_t jc = 0; jc < N; jc += NC) {
    const int64_t nc = std::min<int64_t>(NC, N - jc);
    const int64_t npanels = (nc + NR - 1) / NR;
    for (int64_t pc = 0; pc < K; pc += KC) {
      const int kc = (int)std::min<int64_t>(KC, K - pc);
#pragma omp parallel
      {
#pragma omp for schedule(static) nowait
        for (int64_t jp = 0; jp < npanels; ++jp) {
          float* dst = Bp + jp * NR * KC;
          const int64_t j0 = jc + jp * NR;
          const int nr = (int)std::min<int64_t>(NR, jc + nc - j0);
          for (int k = 0; k < kc; ++k) {
            const float* src = B + (pc + k) * N + j0;
            for (int j = 0; j < nr; ++j) dst[k * NR + j] = src[j];
            for (int j = nr; j < NR; ++j) dst[k * NR + j] = 0.f;
          }
        }
#pragma omp for schedule(static)
        for (int64_t ip = 0; ip < mpanels; ++ip) {
          float* dst = Ap + ip * MR * KC;
          const int64_t i0 = ip * MR;
          const int mr = (int)std::min<int64_t>(MR, M - i0);
          for (int k = 0; k < kc; ++k) {
            for (int i = 0; i < mr; ++i) dst[k * MR + i] = A[(i0 + i) * K + pc + k];
            for (int i = mr; i < MR; ++i) dst[k * MR + i] = 0.f;
          }
        }
#pragma omp for collapse(2) schedule(dynamic, 8)
        for (int64_t jp = 0; jp < npanels; ++jp) {
          for (int64_t ip = 0; ip < mpanels; ++ip) {
            const int64_t i0 = ip * MR, j0 = jc + jp * NR;
            micro_6x16(kc, Ap + ip * MR * KC, Bp + jp * NR * KC, C + i0 * N + j0, N, pc != 0,
                       (int)std::min<int64_t>(MR, M - i0), (int)std::min<int64_t>(NR, jc + nc - j0));
          }
        }
      }
    }
  }
}

// Generic LinalgScalar dot for u32 (wrapping), ndarray.rs:116-122.
void ugemm(int64_t M, int64_t N, int64_t K, const uint32_t* A, const uint32_t* B, uint32_t* C) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      uint32_t acc = 0;
      for (int64_t k = 0; k < K; ++k) acc += A[i * K + k] * B[k * N + j];
      C[i * N + j] = acc;
    }
}

enum BinOp { B_ADD, B_SUB, B_MUL, B_DIV, B_POW, B_LT, B_EQ };

int binary(cgo_ctx* c, int op, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out) {
  if (!a || !b || !out) return fail(c, ST_INVALID, "null argument");
  if (a->dtype != b->dtype) return fail(c, ST_DTYPE, "mixed dtypes in binary operation");
  if (a->shape != b->shape) return fail(c, ST_SHAPE, "Shape mismatch in operation");
  std::unique_ptr<Buf> ha, hb;
  const uint32_t* pa = contig(a, ha);
  const uint32_t* pb = contig(b, hb);
  cgo_tensor* r = fresh(a->dtype, a->shape);
  const int64_t n = r->numel();
  uint32_t* po = r->raw();
  if (a->dtype == DT_F32) {
    const float* x = (const float*)pa;
    const float* y = (const float*)pb;
    float* o = (float*)po;
#pragma omp parallel for schedule(static) if (n > (1 << 15))
    for (int64_t i = 0; i < n; ++i) {
      switch (op) {
        case B_ADD: o[i] = x[i] + y[i]; break;                 // :401-408
        case B_SUB: o[i] = x[i] - y[i]; break;                 // :410-417
        case B_MUL: o[i] = x[i] * y[i]; break;                 // :419-424
        case B_DIV: o[i] = x[i] / y[i]; break;                 // :426-431
        case B_POW: o[i] = powf(x[i], y[i]); break;            // :443-447
        case B_LT: o[i] = x[i] < y[i] ? 1.0f : 0.0f; break;    // :167-172
        case B_EQ: o[i] = x[i] == y[i] ? 1.0f : 0.0f; break;   // :185-190
      }
    }
  } else {
    if (op == B_DIV)
      for (int64_t i = 0; i < n; ++i)
        if (pb[i] == 0) {
          cgo_tensor_release(r);
          return fail(c, ST_INVALID, "attempt to divide by zero");  // Rust panics
        }
#pragma omp parallel for schedule(static) if (n > (1 << 15))
    for (int64_t i = 0; i < n; ++i) {
      switch (op) {
        case B_ADD: po[i] = pa[i] + pb[i]; break;
        case B_SUB: po[i] = pa[i] - pb[i]; break;
        case B_MUL: po[i] = pa[i] * pb[i]; break;
        case B_DIV: po[i] = pa[i] / pb[i]; break;
        case B_POW: po[i] = pow_u32(pa[i], pb[i]); break;      // :449-453
        case B_LT: po[i] = pa[i] < pb[i] ? 1u : 0u; break;     // :173-178
        case B_EQ: po[i] = pa[i] == pb[i] ? 1u : 0u; break;    // :191-196
      }
    }
  }
  *out = r;
  return ST_OK;
}

enum UnOp { U_NEG, U_SIN, U_COS };

int unary(cgo_ctx* c, int op, const cgo_tensor* x, cgo_tensor** out) {
  if (!x || !out) return fail(c, ST_INVALID, "null argument");
  if (op != U_NEG && x->dtype != DT_F32)
    return fail(c, ST_DTYPE, op == U_SIN ? "Invalid input types for sin" : "Invalid input types for cos");
  std::unique_ptr<Buf> hx;
  const uint32_t* px = contig(x, hx);
  cgo_tensor* r = fresh(x->dtype, x->shape);
  const int64_t n = r->numel();
  if (x->dtype == DT_F32) {
    const float* xi = (const float*)px;
    float* o = (float*)r->raw();
#pragma omp parallel for schedule(static) if (n > (1 << 15))
    for (int64_t i = 0; i < n; ++i) {
      switch (op) {
        case U_NEG: o[i] = -xi[i]; break;        // :433-435
        case U_SIN: o[i] = sinf(xi[i]); break;   // :208-214
        case U_COS: o[i] = cosf(xi[i]); break;   // :216-222
      }
    }
  } else {
    uint32_t* o = r->raw();
    for (int64_t i = 0; i < n; ++i) o[i] = 0u - px[i];  // wrapping_neg, :437-441
  }
  *out = r;
  return ST_OK;
}

enum RedOp { R_SUM, R_MAX, R_ARGMAX };

int reduce(cgo_ctx* c, int op, const cgo_tensor* x, cgo_tensor** out) {
  if (!x || !out) return fail(c, ST_INVALID, "null argument");
  const int r = (int)x->shape.size();
  if (r == 0) {
    // The shape-only backend leaves rank-0 inputs unchanged (shape_only.rs:304-315).
    cgo_tensor* t = fresh(op == R_ARGMAX ? DT_U32 : x->dtype, {});
    t->raw()[0] = op == R_ARGMAX ? 0u : x->raw()[0];
    *out = t;
    return ST_OK;
  }
  const int64_t n = x->shape[r - 1];
  if (op == R_ARGMAX && n == 0) return fail(c, ST_SHAPE, "argmax over an empty axis");
  std::unique_ptr<Buf> hx;
  const uint32_t* px = contig(x, hx);
  std::vector<int64_t> oshape = x->shape;
  oshape[r - 1] = 1;
  cgo_tensor* t = fresh(op == R_ARGMAX ? DT_U32 : x->dtype, oshape);
  const int64_t rows = t->numel();
  uint32_t* po = t->raw();
#pragma omp parallel for schedule(static) if (rows * n > (1 << 15))
  for (int64_t row = 0; row < rows; ++row) {
    const uint32_t* lane = px + row * n;
    if (x->dtype == DT_F32) {
      const float* f = (const float*)lane;
      if (op == R_SUM) {
        po[row] = asu(lane_sum<float>(f, n));                     // :522-529
      } else if (op == R_MAX) {
        float acc = -3.4028234663852886e38f;                      // f32::MIN, :455-460
        for (int64_t i = 0; i < n; ++i) acc = fmaxf(acc, f[i]);   // f32::max ignores NaN
        po[row] = asu(acc);
      } else {
        // max_by(total_cmp) keeps the LAST maximal element, :469-480
        uint32_t bestk = 0, besti = 0;
        for (int64_t i = 0; i < n; ++i) {
          uint32_t k = total_key(lane[i]);
          if (i == 0 || k >= bestk) { bestk = k; besti = (uint32_t)i; }
        }
        po[row] = besti;
      }
    } else {
      if (op == R_SUM) {
        po[row] = lane_sum<uint32_t>(lane, n);
      } else if (op == R_MAX) {
        uint32_t acc = 0;                                         // u32::MIN, :462-467
        for (int64_t i = 0; i < n; ++i) acc = std::max(acc, lane[i]);
        po[row] = acc;
      } else {
        uint32_t best = 0, besti = 0;                             // :482-493
        for (int64_t i = 0; i < n; ++i)
          if (i == 0 || lane[i] >= best) { best = lane[i]; besti = (uint32_t)i; }
        po[row] = besti;
      }
    }
  }
  *out = t;
  return ST_OK;
}

}  // namespace

extern "C" {

int32_t cgo_ctx_create(int32_t threads, cgo_ctx** out) {
  if (!out) return ST_INVALID;
  auto* c = new cgo_ctx();
#ifdef _OPENMP
  c->threads = threads > 0 ? threads : omp_get_num_procs();
  omp_set_num_threads(c->threads);
#else
  (void)threads;
  c->threads = 1;
#endif
  *out = c;
  return ST_OK;
}
int32_t cgo_ctx_destroy(cgo_ctx* c) { delete c; return ST_OK; }
const char* cgo_last_error(cgo_ctx* c) { return c ? c->err.c_str() : ""; }
int32_t cgo_ctx_threads(cgo_ctx* c) { return c ? c->threads : 0; }

int32_t cgo_tensor_retain(cgo_tensor* t) { if (!t) return ST_INVALID; t->rc++; return ST_OK; }
int32_t cgo_tensor_release(cgo_tensor* t) {
  if (!t) return ST_INVALID;
  if (--t->rc == 0) delete t;
  return ST_OK;
}
// BackendTensorOps::shape, :618-628
int32_t cgo_shape(const cgo_tensor* t, int32_t* rank, int64_t dims[8]) {
  if (!t || !rank || !dims) return ST_INVALID;
  *rank = (int32_t)t->shape.size();
  for (size_t i = 0; i < t->shape.size(); ++i) dims[i] = t->shape[i];
  return ST_OK;
}
int32_t cgo_dtype_of(const cgo_tensor* t, int32_t* dtype) {
  if (!t || !dtype) return ST_INVALID;
  *dtype = t->dtype;
  return ST_OK;
}

// :53-65
int32_t cgo_zeros(cgo_ctx* c, const int64_t* dims, int32_t rank, int32_t dtype, cgo_tensor** out) {
  if (!out || rank < 0 || rank > 8 || (rank && !dims)) return fail(c, ST_INVALID, "bad argument");
  cgo_tensor* t = fresh(dtype, std::vector<int64_t>(dims, dims + rank));
  memset(t->raw(), 0, (size_t)t->numel() * 4);
  *out = t;
  return ST_OK;
}

static int from_vec(cgo_ctx* c, int dtype, const void* data, int64_t n, const int64_t* dims,
                    int32_t rank, cgo_tensor** out) {
  if (!out || rank < 0 || rank > 8 || (rank && !dims)) return fail(c, ST_INVALID, "bad argument");
  std::vector<int64_t> shape(dims, dims + rank);
  int64_t want = 1;
  for (auto d : shape) want *= d;
  if (want != n) return fail(c, ST_SHAPE, "ShapeError");  // from_shape_vec fails, :73-74
  cgo_tensor* t = fresh(dtype, shape);
  if (n) memcpy(t->raw(), data, (size_t)n * 4);
  *out = t;
  return ST_OK;
}
// :67-77
int32_t cgo_ndarray_from_vec_f32(cgo_ctx* c, const float* d, int64_t n, const int64_t* dims, int32_t rank, cgo_tensor** out) {
  return from_vec(c, DT_F32, d, n, dims, rank, out);
}
// :79-89
int32_t cgo_ndarray_from_vec_u32(cgo_ctx* c, const uint32_t* d, int64_t n, const int64_t* dims, int32_t rank, cgo_tensor** out) {
  return from_vec(c, DT_U32, d, n, dims, rank, out);
}

// :97-114
int32_t cgo_cast(cgo_ctx* c, const cgo_tensor* x, int32_t dtype, cgo_tensor** out) {
  if (!x || !out) return fail(c, ST_INVALID, "null argument");
  if (x->dtype == dtype) {  // identity arms return the same value
    cgo_tensor_retain(const_cast<cgo_tensor*>(x));
    *out = const_cast<cgo_tensor*>(x);
    return ST_OK;
  }
  std::unique_ptr<Buf> hx;
  const uint32_t* px = contig(x, hx);
  cgo_tensor* t = fresh(dtype, x->shape);
  const int64_t n = t->numel();
  if (dtype == DT_U32) {
    const float* f = (const float*)px;
    for (int64_t i = 0; i < n; ++i) t->raw()[i] = f32_as_u32(f[i]);
  } else {
    float* o = (float*)t->raw();
    for (int64_t i = 0; i < n; ++i) o[i] = (float)px[i];
  }
  *out = t;
  return ST_OK;
}

// :116-122 and :531-615
int32_t cgo_matmul(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** out) {
  if (!a || !b || !out) return fail(c, ST_INVALID, "null argument");
  if (a->dtype != b->dtype) return fail(c, ST_DTYPE, "mixed dtypes in matmul");
  const int ra = (int)a->shape.size(), rb = (int)b->shape.size();
  if (ra < 2) return fail(c, ST_SHAPE, "batched_matmul: lhs must be at least rank 2");
  if (rb < 2) return fail(c, ST_SHAPE, "batched_matmul: rhs must be at least rank 2");
  const int64_t M = a->shape[ra - 2], K = a->shape[ra - 1], K2 = b->shape[rb - 2], N = b->shape[rb - 1];
  if (K != K2) return fail(c, ST_SHAPE, "batched_matmul: incompatible matrix dimensions");
  std::vector<int64_t> ba(a->shape.begin(), a->shape.end() - 2), bb(b->shape.begin(), b->shape.end() - 2);
  if (ba != bb) return fail(c, ST_SHAPE, "batched_matmul: batch dimensions must match");
  int64_t batch = 1;
  for (auto d : ba) batch *= d;
  std::unique_ptr<Buf> ha, hb;
  const uint32_t* pa = contig(a, ha);  // to_shape((batch,m,k)) of a non-standard layout copies
  const uint32_t* pb = contig(b, hb);
  std::vector<int64_t> oshape = ba;
  oshape.push_back(M);
  oshape.push_back(N);
  cgo_tensor* t = fresh(a->dtype, oshape);
  for (int64_t i = 0; i < batch; ++i) {
    if (a->dtype == DT_F32)
      sgemm(M, N, K, (const float*)pa + i * M * K, (const float*)pb + i * K * N, (float*)t->raw() + i * M * N);
    else
      ugemm(M, N, K, pa + i * M * K, pb + i * K * N, t->raw() + i * M * N);
  }
  *out = t;
  return ST_OK;
}

int32_t cgo_add(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_ADD, a, b, o); }
int32_t cgo_sub(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_SUB, a, b, o); }
int32_t cgo_mul(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_MUL, a, b, o); }
int32_t cgo_div(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_DIV, a, b, o); }
int32_t cgo_pow(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_POW, a, b, o); }
int32_t cgo_lt(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_LT, a, b, o); }
int32_t cgo_eq(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, cgo_tensor** o) { return binary(c, B_EQ, a, b, o); }
int32_t cgo_sin(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return unary(c, U_SIN, x, o); }
int32_t cgo_cos(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return unary(c, U_COS, x, o); }
int32_t cgo_neg(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return unary(c, U_NEG, x, o); }
int32_t cgo_max(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return reduce(c, R_MAX, x, o); }
int32_t cgo_sum(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return reduce(c, R_SUM, x, o); }
int32_t cgo_argmax(cgo_ctx* c, const cgo_tensor* x, cgo_tensor** o) { return reduce(c, R_ARGMAX, x, o); }

// :259-265, :355-361 — numpy right-aligned broadcast, then to_owned() materialises.
int32_t cgo_broadcast(cgo_ctx* c, const cgo_tensor* x, const int64_t* dims, int32_t rank, cgo_tensor** out) {
  if (!x || !out || rank < 0 || rank > 8 || (rank && !dims)) return fail(c, ST_INVALID, "bad argument");
  const int rx = (int)x->shape.size();
  if (rx > rank) return fail(c, ST_SHAPE, "broadcast: target has lower rank");
  cgo_tensor v;
  v.dtype = x->dtype;
  v.buf = x->buf;
  v.offset = x->offset;
  v.shape.assign(dims, dims + rank);
  v.strides.assign(rank, 0);
  for (int i = 0; i < rx; ++i) {
    const int o = rank - rx + i;
    if (x->shape[i] == dims[o]) v.strides[o] = x->strides[i];
    else if (x->shape[i] == 1) v.strides[o] = 0;
    else return fail(c, ST_SHAPE, "broadcast: incompatible shapes");
  }
  cgo_tensor* t = fresh(x->dtype, v.shape);
  gather(&v, t->raw());
  *out = t;
  return ST_OK;
}

// :311-317, :347-353 — to_shape in logical row-major order, then to_owned().
int32_t cgo_reshape(cgo_ctx* c, const cgo_tensor* x, const int64_t* dims, int32_t rank, cgo_tensor** out) {
  if (!x || !out || rank < 0 || rank > 8 || (rank && !dims)) return fail(c, ST_INVALID, "bad argument");
  std::vector<int64_t> shape(dims, dims + rank);
  int64_t n = 1;
  for (auto d : shape) n *= d;
  if (n != x->numel()) return fail(c, ST_SHAPE, "reshape: element count differs");
  cgo_tensor* t = fresh(x->dtype, shape);
  gather(x, t->raw());
  *out = t;
  return ST_OK;
}

// :267-273, :363-371 — copy, then swap_axes: the result is a non-contiguous array.
int32_t cgo_transpose(cgo_ctx* c, const cgo_tensor* x, int32_t d0, int32_t d1, cgo_tensor** out) {
  if (!x || !out) return fail(c, ST_INVALID, "null argument");
  const int r = (int)x->shape.size();
  if (d0 < 0 || d1 < 0 || d0 >= r || d1 >= r) return fail(c, ST_SHAPE, "transpose: axis out of range");
  cgo_tensor* t = fresh(x->dtype, x->shape);
  gather(x, t->raw());
  std::swap(t->shape[d0], t->shape[d1]);
  std::swap(t->strides[d0], t->strides[d1]);
  *out = t;
  return ST_OK;
}

// :248-257, :495-520 — stable sort of indices by descending total order, first k.
int32_t cgo_topk(cgo_ctx* c, const cgo_tensor* x, int64_t k, cgo_tensor** values, cgo_tensor** indices) {
  if (!x || !values || !indices) return fail(c, ST_INVALID, "null argument");
  if (x->dtype != DT_F32) return fail(c, ST_DTYPE, "Unsupported type for topk");
  const int r = (int)x->shape.size();
  if (r == 0) return fail(c, ST_SHAPE, "topk of a rank-0 tensor");
  const int64_t n = x->shape[r - 1];
  if (k < 0 || k > n) return fail(c, ST_SHAPE, "topk: k exceeds the last dimension");
  std::unique_ptr<Buf> hx;
  const uint32_t* px = contig(x, hx);
  std::vector<int64_t> oshape = x->shape;
  oshape[r - 1] = k;
  cgo_tensor* tv = fresh(DT_F32, oshape);
  cgo_tensor* ti = fresh(DT_U32, oshape);
  const int64_t rows = n ? x->numel() / n : 0;
  std::vector<uint32_t> idx((size_t)n);
  for (int64_t row = 0; row < rows; ++row) {
    const uint32_t* lane = px + row * n;
    std::iota(idx.begin(), idx.end(), 0u);
    std::stable_sort(idx.begin(), idx.end(),
                     [&](uint32_t i, uint32_t j) { return total_key(lane[i]) > total_key(lane[j]); });
    for (int64_t j = 0; j < k; ++j) {
      tv->raw()[row * k + j] = lane[idx[j]];
      ti->raw()[row * k + j] = idx[j];
    }
  }
  *values = tv;
  *indices = ti;
  return ST_OK;
}

// :337-343 — ArcArray == : same shape and every element ==
int32_t cgo_compare(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, int32_t* equal) {
  if (!a || !b || !equal) return fail(c, ST_INVALID, "null argument");
  if (a->dtype != b->dtype) return fail(c, ST_DTYPE, "mixed dtypes in compare");
  *equal = 0;
  if (a->shape != b->shape) return ST_OK;
  std::unique_ptr<Buf> ha, hb;
  const uint32_t* pa = contig(a, ha);
  const uint32_t* pb = contig(b, hb);
  const int64_t n = a->numel();
  for (int64_t i = 0; i < n; ++i) {
    if (a->dtype == DT_F32) { if (!(asf(pa[i]) == asf(pb[i]))) return ST_OK; }
    else if (pa[i] != pb[i]) return ST_OK;
  }
  *equal = 1;
  return ST_OK;
}

// :319-335, :393-399
int32_t cgo_concat(cgo_ctx* c, const cgo_tensor* a, const cgo_tensor* b, int32_t dim, cgo_tensor** out) {
  if (!a || !b || !out) return fail(c, ST_INVALID, "null argument");
  if (a->dtype != b->dtype) return fail(c, ST_DTYPE, "Incompatible types for concatenation");
  const int r = (int)a->shape.size();
  if ((int)b->shape.size() != r || dim < 0 || dim >= r) return fail(c, ST_SHAPE, "concat: rank or axis mismatch");
  for (int i = 0; i < r; ++i)
    if (i != dim && a->shape[i] != b->shape[i]) return fail(c, ST_SHAPE, "concat: shapes differ off the axis");
  std::unique_ptr<Buf> ha, hb;
  const uint32_t* pa = contig(a, ha);
  const uint32_t* pb = contig(b, hb);
  std::vector<int64_t> oshape = a->shape;
  oshape[dim] += b->shape[dim];
  cgo_tensor* t = fresh(a->dtype, oshape);
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < dim; ++i) outer *= a->shape[i];
  for (int i = dim + 1; i < r; ++i) inner *= a->shape[i];
  const int64_t ca = a->shape[dim] * inner, cb = b->shape[dim] * inner;
  for (int64_t o = 0; o < outer; ++o) {
    memcpy(t->raw() + o * (ca + cb), pa + o * ca, (size_t)ca * 4);
    memcpy(t->raw() + o * (ca + cb) + ca, pb + o * cb, (size_t)cb * 4);
  }
  *out = t;
  return ST_OK;
}

// :275-295, :373-381 — select(Axis(dim), flattened indices)
int32_t cgo_index(cgo_ctx* c, const cgo_tensor* x, int32_t dim, const cgo_tensor* indices, cgo_tensor** out) {
  if (!x || !indices || !out) return fail(c, ST_INVALID, "null argument");
  if (indices->dtype != DT_U32) return fail(c, ST_DTYPE, "Invalid input types for indexing");
  const int r = (int)x->shape.size();
  if (dim < 0 || dim >= r) return fail(c, ST_SHAPE, "index: axis out of range");
  std::unique_ptr<Buf> hx, hi;
  const uint32_t* px = contig(x, hx);
  const uint32_t* pi = contig(indices, hi);
  const int64_t ni = indices->numel();
  for (int64_t i = 0; i < ni; ++i)
    if ((int64_t)pi[i] >= x->shape[dim]) return fail(c, ST_INDEX, "index out of bounds");
  std::vector<int64_t> oshape = x->shape;
  oshape[dim] = ni;
  cgo_tensor* t = fresh(x->dtype, oshape);
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < dim; ++i) outer *= x->shape[i];
  for (int i = dim + 1; i < r; ++i) inner *= x->shape[i];
  const int64_t xd = x->shape[dim];
#pragma omp parallel for collapse(2) schedule(static) if (outer * ni * inner > (1 << 16))
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t j = 0; j < ni; ++j)
      memcpy(t->raw() + (o * ni + j) * inner, px + (o * xd + pi[j]) * inner, (size_t)inner * 4);
  *out = t;
  return ST_OK;
}

// :297-309, :383-391 — slice_axis(...).to_owned()
int32_t cgo_slice(cgo_ctx* c, const cgo_tensor* x, int32_t dim, int64_t start, int64_t len, cgo_tensor** out) {
  if (!x || !out) return fail(c, ST_INVALID, "null argument");
  const int r = (int)x->shape.size();
  if (dim < 0 || dim >= r) return fail(c, ST_SHAPE, "slice: axis out of range");
  if (start < 0 || len < 0 || start + len > x->shape[dim]) return fail(c, ST_SHAPE, "slice: range out of bounds");
  cgo_tensor v;
  v.dtype = x->dtype;
  v.buf = x->buf;
  v.shape = x->shape;
  v.strides = x->strides;
  v.shape[dim] = len;
  v.offset = x->offset + start * x->strides[dim];
  cgo_tensor* t = fresh(x->dtype, v.shape);
  gather(&v, t->raw());
  *out = t;
  return ST_OK;
}

// :91-95 — Array::range(0.0, end as f32, 1.0) then cast to u32
int32_t cgo_arange(cgo_ctx* c, int64_t end, cgo_tensor** out) {
  if (!out || end < 0) return fail(c, ST_INVALID, "bad argument");
  const int64_t n = (int64_t)ceilf((float)end);
  cgo_tensor* t = fresh(DT_U32, {n});
  for (int64_t i = 0; i < n; ++i) t->raw()[i] = f32_as_u32(0.0f + 1.0f * (float)i);
  *out = t;
  return ST_OK;
}

// :46-51 — as_slice().unwrap(): a non-standard layout panics in the reference
static int to_vec(cgo_ctx* c, int dtype, const cgo_tensor* x, void* dst, int64_t n) {
  if (!x || (!dst && n)) return fail(c, ST_INVALID, "null argument");
  if (x->dtype != dtype) return fail(c, ST_DTYPE, "to_vec: dtype tag differs");
  if (n != x->numel()) return fail(c, ST_SHAPE, "to_vec: element count differs");
  if (!x->contiguous()) return fail(c, ST_SHAPE, "to_vec: array is not in standard layout");
  if (n) memcpy(dst, x->raw(), (size_t)n * 4);
  return ST_OK;
}
int32_t cgo_to_vec_f32(cgo_ctx* c, const cgo_tensor* x, float* dst, int64_t n) { return to_vec(c, DT_F32, x, dst, n); }
int32_t cgo_to_vec_u32(cgo_ctx* c, const cgo_tensor* x, uint32_t* dst, int64_t n) { return to_vec(c, DT_U32, x, dst, n); }

}  // extern "C"
