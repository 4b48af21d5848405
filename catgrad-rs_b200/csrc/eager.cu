// eager.cu — the trait methods that launch kernels, one launch per call: strided
// elementwise maps, last-axis reductions, argmax/top-k, gathers and copies, and the f32
// CUDA-core GEMM that serves as the exact-precision path.  Inputs are arbitrary strided
// views (broadcast = stride 0, transpose = swapped strides); outputs are contiguous.
#include "runtime.h"

#include <algorithm>
#include <cstring>

namespace cg {

// ------------------------------------------------------------------ device helpers ---

__device__ __forceinline__ float ld_f(const void* p, int st, int64_t i) {
  return st == ST_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ uint32_t ld_u(const void* p, int64_t i) { return ((const uint32_t*)p)[i]; }

// Rust `f32 as u32`: saturating, NaN -> 0.
__device__ __forceinline__ uint32_t f32_as_u32(float v) {
  if (!(v == v) || v <= 0.f) return 0u;
  if (v >= 4294967296.f) return 0xFFFFFFFFu;
  return (uint32_t)v;
}
// Orders f32 bit patterns like Rust's f32::total_cmp.
__device__ __forceinline__ uint32_t total_key(uint32_t b) { return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }

__device__ __forceinline__ uint32_t pow_u32(uint32_t a, uint32_t b) {
  uint32_t r = 1;
  while (b) {
    if (b & 1) r *= a;
    a *= a;
    b >>= 1;
  }
  return r;
}

// Offsets of linear index i in up to three operands.
__device__ __forceinline__ void offsets(const Iter& it, int64_t i, int64_t& o0, int64_t& o1, int64_t& o2) {
  o0 = o1 = o2 = 0;
#pragma unroll 1
  for (int d = it.rank - 1; d >= 0; --d) {
    int64_t q = i / it.dims[d];
    int64_t r = i - q * it.dims[d];
    o0 += r * it.s0[d];
    o1 += r * it.s1[d];
    o2 += r * it.s2[d];
    i = q;
  }
}

enum { OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_POW, OP_LT, OP_EQ };
enum { UN_NEG, UN_SIN, UN_COS };

template <int OP>
__device__ __forceinline__ float apply_f(float a, float b) {
  if (OP == OP_ADD) return a + b;
  if (OP == OP_SUB) return a - b;
  if (OP == OP_MUL) return a * b;
  if (OP == OP_DIV) return a / b;
  // powf of the host libm is (nearly) correctly rounded; going through double keeps the
  // device within one ulp of it
  if (OP == OP_POW) return (float)pow((double)a, (double)b);
  if (OP == OP_LT) return a < b ? 1.f : 0.f;
  return a == b ? 1.f : 0.f;
}
template <int OP>
__device__ __forceinline__ uint32_t apply_u(uint32_t a, uint32_t b) {
  if (OP == OP_ADD) return a + b;
  if (OP == OP_SUB) return a - b;
  if (OP == OP_MUL) return a * b;
  if (OP == OP_DIV) return b ? a / b : 0xFFFFFFFFu;
  if (OP == OP_POW) return pow_u32(a, b);
  if (OP == OP_LT) return a < b ? 1u : 0u;
  return a == b ? 1u : 0u;
}

template <int OP>
__global__ void k_binary_f32(Iter it, const void* a, int sta, const void* b, int stb, float* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t oa, ob, oc;
    offsets(it, i, oa, ob, oc);
    out[i] = apply_f<OP>(ld_f(a, sta, oa), ld_f(b, stb, ob));
  }
}
// both operands contiguous f32, 16-byte aligned: 128-bit loads and stores
template <int OP>
__global__ void k_binary_f32_vec(const float4* a, const float4* b, float4* out, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 x = a[i], y = b[i], r;
    r.x = apply_f<OP>(x.x, y.x);
    r.y = apply_f<OP>(x.y, y.y);
    r.z = apply_f<OP>(x.z, y.z);
    r.w = apply_f<OP>(x.w, y.w);
    out[i] = r;
  }
}
template <int OP>
__global__ void k_binary_u32(Iter it, const uint32_t* a, const uint32_t* b, uint32_t* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t oa, ob, oc;
    offsets(it, i, oa, ob, oc);
    out[i] = apply_u<OP>(a[oa], b[ob]);
  }
}

template <int OP>
__global__ void k_unary_f32(Iter it, const void* x, int st, float* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t o0, o1, o2;
    offsets(it, i, o0, o1, o2);
    float v = ld_f(x, st, o0);
    if (OP == UN_NEG) out[i] = -v;
    else if (OP == UN_SIN) out[i] = (float)sin((double)v);
    else out[i] = (float)cos((double)v);
  }
}
__global__ void k_neg_u32(Iter it, const uint32_t* x, uint32_t* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t o0, o1, o2;
    offsets(it, i, o0, o1, o2);
    out[i] = 0u - x[o0];
  }
}

// strided copy; mode 0: 4-byte words, 1: bf16 -> bf16, 2: bf16 -> f32, 3: f32 -> bf16,
// 4: f32 -> u32 (Rust `as`), 5: u32 -> f32.  dst is addressed with s1 (so it may be a view).
template <int MODE>
__global__ void k_copy(Iter it, const void* src, void* dst, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t o0, o1, o2;
    offsets(it, i, o0, o1, o2);
    if (MODE == 0) ((uint32_t*)dst)[o1] = ((const uint32_t*)src)[o0];
    else if (MODE == 1) ((__nv_bfloat16*)dst)[o1] = ((const __nv_bfloat16*)src)[o0];
    else if (MODE == 2) ((float*)dst)[o1] = __bfloat162float(((const __nv_bfloat16*)src)[o0]);
    else if (MODE == 3) ((__nv_bfloat16*)dst)[o1] = __float2bfloat16_rn(((const float*)src)[o0]);
    else if (MODE == 4) ((uint32_t*)dst)[o1] = f32_as_u32(((const float*)src)[o0]);
    else ((float*)dst)[o1] = (float)((const uint32_t*)src)[o0];
  }
}

__global__ void k_arange(uint32_t* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = f32_as_u32(0.0f + 1.0f * (float)i);
}

// ------------------------------------------------------------------ reductions -------
enum { RED_SUM, RED_MAX, RED_ARGMAX };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
    v = w > v ? w : v;
  }
  return v;
}

// One block per row of a contiguous [rows, n] array.  `isf` selects f32 or u32 semantics.
template <int RED>
__global__ void k_reduce_rows(const void* x, int st, int isf, uint32_t* out, int64_t n) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  __shared__ unsigned long long sh64[32];
  __shared__ float shf[32];
  __shared__ uint32_t shu[32];
  if (RED == RED_SUM) {
    if (isf) {
      float acc = 0.f;
      for (int64_t i = tid; i < n; i += blockDim.x) acc += ld_f(x, st, row * n + i);
      acc = warp_sum(acc);
      if (lane == 0) shf[wid] = acc;
      __syncthreads();
      if (wid == 0) {
        acc = lane < nw ? shf[lane] : 0.f;
        acc = warp_sum(acc);
        if (lane == 0) ((float*)out)[row] = acc;
      }
    } else {
      uint32_t acc = 0;
      for (int64_t i = tid; i < n; i += blockDim.x) acc += ld_u(x, row * n + i);
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) shu[wid] = acc;
      __syncthreads();
      if (wid == 0) {
        acc = lane < nw ? shu[lane] : 0u;
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[row] = acc;
      }
    }
  } else if (RED == RED_MAX) {
    if (isf) {
      float acc = -3.4028234663852886e38f;  // f32::MIN; fmaxf drops NaN like f32::max
      for (int64_t i = tid; i < n; i += blockDim.x) acc = fmaxf(acc, ld_f(x, st, row * n + i));
      for (int o = 16; o; o >>= 1) acc = fmaxf(acc, __shfl_xor_sync(0xffffffffu, acc, o));
      if (lane == 0) shf[wid] = acc;
      __syncthreads();
      if (wid == 0) {
        acc = lane < nw ? shf[lane] : -3.4028234663852886e38f;
        for (int o = 16; o; o >>= 1) acc = fmaxf(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if (lane == 0) ((float*)out)[row] = acc;
      }
    } else {
      uint32_t acc = 0;
      for (int64_t i = tid; i < n; i += blockDim.x) acc = max(acc, ld_u(x, row * n + i));
      for (int o = 16; o; o >>= 1) acc = max(acc, __shfl_xor_sync(0xffffffffu, acc, o));
      if (lane == 0) shu[wid] = acc;
      __syncthreads();
      if (wid == 0) {
        acc = lane < nw ? shu[lane] : 0u;
        for (int o = 16; o; o >>= 1) acc = max(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if (lane == 0) out[row] = acc;
      }
    }
  } else {
    // (key << 32) | index: the maximum is the greatest key and, among equals, the LAST index
    unsigned long long best = 0;
    for (int64_t i = tid; i < n; i += blockDim.x) {
      uint32_t bits = isf ? __float_as_uint(ld_f(x, st, row * n + i)) : ld_u(x, row * n + i);
      uint32_t key = isf ? total_key(bits) : bits;
      unsigned long long v = ((unsigned long long)key << 32) | (uint32_t)i;
      best = v > best ? v : best;
    }
    best = warp_max_u64(best);
    if (lane == 0) sh64[wid] = best;
    __syncthreads();
    if (wid == 0) {
      best = lane < nw ? sh64[lane] : 0ull;
      best = warp_max_u64(best);
      if (lane == 0) out[row] = (uint32_t)(best & 0xFFFFFFFFull);
    }
  }
}

// arg-max of each row of a contiguous f32 [rows, n], n a multiple of 4, rows 16-byte aligned:
// 128-bit loads, and the running maximum kept as a 32-bit total-order key plus an index (a later
// index wins ties, and every thread meets its elements in ascending index order, so `>=` keeps
// the last one); the 64-bit (key, index) pairs only meet in the final merges.
__global__ void k_argmax_rows_f32(const float* x, uint32_t* out, int64_t n) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  __shared__ unsigned long long sh64[32];
  const uint4* r4 = (const uint4*)(x + row * n);
  const int n4 = (int)(n / 4);
  uint32_t bk = 0, bi = 0;
  bool any = false;
  for (int i = tid; i < n4; i += blockDim.x) {
    const uint4 v = r4[i];
    const uint32_t k0 = total_key(v.x), k1 = total_key(v.y), k2 = total_key(v.z), k3 = total_key(v.w);
    // the last of the four that attains their maximum
    uint32_t k = k0, j = 0;
    if (k1 >= k) { k = k1; j = 1; }
    if (k2 >= k) { k = k2; j = 2; }
    if (k3 >= k) { k = k3; j = 3; }
    if (!any || k >= bk) { bk = k; bi = (uint32_t)i * 4u + j; any = true; }
  }
  unsigned long long best = any ? (((unsigned long long)bk << 32) | bi) : 0ull;
  best = warp_max_u64(best);
  if (lane == 0) sh64[wid] = best;
  __syncthreads();
  if (wid == 0) {
    best = lane < nw ? sh64[lane] : 0ull;
    best = warp_max_u64(best);
    if (lane == 0) out[row] = (uint32_t)(best & 0xFFFFFFFFull);
  }
}

// top-k of each row of a contiguous f32 [rows, n]: k rounds of "largest key below the last
// one taken", key = (total order key << 32) | ~index, so equal values come out in
// ascending index order like a stable descending sort.
__global__ void k_topk_rows(const float* x, float* vals, uint32_t* idx, int64_t n, int64_t k) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  __shared__ unsigned long long sh[32];
  __shared__ unsigned long long chosen;
  unsigned long long bound = ~0ull;
  bool first = true;
  for (int64_t j = 0; j < k; ++j) {
    unsigned long long best = 0;
    bool have = false;
    for (int64_t i = tid; i < n; i += blockDim.x) {
      uint32_t key = total_key(__float_as_uint(x[row * n + i]));
      unsigned long long v = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
      if ((first || v < bound) && (!have || v > best)) { best = v; have = true; }
    }
    // 0 is a legal key only for index 0xFFFFFFFF of a -NaN; rows that long are rejected by the host
    best = warp_max_u64(have ? best : 0ull);
    if (lane == 0) sh[wid] = best;
    __syncthreads();
    if (wid == 0) {
      best = lane < nw ? sh[lane] : 0ull;
      best = warp_max_u64(best);
      if (lane == 0) chosen = best;
    }
    __syncthreads();
    bound = chosen;
    first = false;
    if (tid == 0) {
      uint32_t i = ~(uint32_t)(bound & 0xFFFFFFFFull);
      idx[row * k + j] = i;
      vals[row * k + j] = x[row * n + i];
    }
    __syncthreads();
  }
}

// out[o, j, i] = x[o, idx[j], i] on contiguous x; a bad index raises the context's error
// word and reads row 0.
__global__ void k_index(const uint32_t* x, const uint32_t* idx, uint32_t* out, int64_t outer, int64_t xd,
                        int64_t ni, int64_t inner, int32_t* err) {
  const int64_t n = outer * ni * inner;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t in = i % inner, t = i / inner;
    int64_t j = t % ni, o = t / ni;
    uint32_t r = idx[j];
    if (r >= xd) { *err = DEV_INDEX; r = 0; }
    out[i] = x[(o * xd + r) * inner + in];
  }
}
// The same when a gathered row (`inner` elements) is a whole number of 16-byte vectors: one block
// per output row copies it with 128-bit loads and stores; no per-element index arithmetic.
// row_vecs = bytes of a row / 16.
__global__ void k_index_rows(const uint4* x, const uint32_t* idx, uint4* out, int64_t xd, int64_t ni, int64_t rows,
                             int64_t row_vecs, int32_t* err) {
  for (int64_t t = blockIdx.x; t < rows; t += gridDim.x) {
    const int64_t j = t % ni, o = t / ni;
    uint32_t r = idx[j];
    if (r >= xd) { if (threadIdx.x == 0) *err = DEV_INDEX; r = 0; }
    const uint4* src = x + (o * xd + r) * row_vecs;
    uint4* dst = out + t * row_vecs;
    for (int64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) dst[i] = src[i];
  }
}
// same for 2-byte elements
__global__ void k_index16(const uint16_t* x, const uint32_t* idx, uint16_t* out, int64_t outer, int64_t xd,
                          int64_t ni, int64_t inner, int32_t* err) {
  const int64_t n = outer * ni * inner;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t in = i % inner, t = i / inner;
    int64_t j = t % ni, o = t / ni;
    uint32_t r = idx[j];
    if (r >= xd) { *err = DEV_INDEX; r = 0; }
    out[i] = x[(o * xd + r) * inner + in];
  }
}

// whole-array equality: result word stays 1 unless some pair differs
__global__ void k_compare(Iter it, const void* a, int sta, const void* b, int stb, int isf, int64_t n, int32_t* res) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t oa, ob, oc;
    offsets(it, i, oa, ob, oc);
    bool same = isf ? (ld_f(a, sta, oa) == ld_f(b, stb, ob)) : (ld_u(a, oa) == ld_u(b, ob));
    if (!same) *res = 0;
  }
}

// ------------------------------------------------------------------ f32 / u32 GEMM ---
// C[z] = A[z] B[z] with arbitrary element strides, 64x64 tile, 16-deep k step, 4x4 per
// thread, plain FMA accumulation in k order (the exact-f32 path).
struct GemmArgs {
  const void* a;
  const void* b;
  void* c;
  int sta, stb;
  int64_t M, N, K;
  int64_t a_m, a_k, b_k, b_n;
  int nb;  // batch dims
  int64_t bd[CG_MAX_RANK], ba[CG_MAX_RANK], bb[CG_MAX_RANK];
};

template <typename T>
__global__ void __launch_bounds__(256) k_gemm_simt(GemmArgs g) {
  __shared__ T As[16][64 + 4];
  __shared__ T Bs[16][64 + 4];
  int64_t z = blockIdx.z, oa = 0, ob = 0;
  for (int d = g.nb - 1; d >= 0; --d) {
    int64_t q = z / g.bd[d], r = z - q * g.bd[d];
    oa += r * g.ba[d];
    ob += r * g.bb[d];
    z = q;
  }
  const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;
  // pick the thread->element map that walks the unit-stride direction
  const bool a_kfast = g.a_k == 1 || g.a_m != 1;
  const bool b_nfast = g.b_n == 1 || g.b_k != 1;
  for (int64_t k0 = 0; k0 < g.K; k0 += 16) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int e = tid + r * 256;  // 1024 elements of a 64x16 tile
      int mm, kk;
      if (a_kfast) { kk = e & 15; mm = e >> 4; } else { mm = e & 63; kk = e >> 6; }
      int64_t m = m0 + mm, k = k0 + kk;
      T v = 0;
      if (m < g.M && k < g.K) {
        int64_t o = oa + m * g.a_m + k * g.a_k;
        if (sizeof(T) == 4 && g.sta == ST_BF16) v = (T)__bfloat162float(((const __nv_bfloat16*)g.a)[o]);
        else v = ((const T*)g.a)[o];
      }
      As[kk][mm] = v;
      int nn;
      if (b_nfast) { nn = e & 63; kk = e >> 6; } else { kk = e & 15; nn = e >> 4; }
      int64_t n = n0 + nn;
      k = k0 + kk;
      v = 0;
      if (n < g.N && k < g.K) {
        int64_t o = ob + k * g.b_k + n * g.b_n;
        if (sizeof(T) == 4 && g.stb == ST_BF16) v = (T)__bfloat162float(((const __nv_bfloat16*)g.b)[o]);
        else v = ((const T*)g.b)[o];
      }
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      T av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
  T* c = (T*)g.c + (int64_t)blockIdx.z * g.M * g.N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t n = n0 + tx * 4 + j;
      if (n < g.N) c[m * g.N + n] = acc[i][j];
    }
  }
}

// ------------------------------------------------------------------ host helpers -----

static int copy_into(cg_ctx* c, const cg_tensor* src, void* dst, int dst_storage, const int64_t* dst_strides,
                     int mode_override = -1) {
  const int64_t n = src->numel();
  if (n == 0) return CG_OK;
  Iter it = make_iter(src->rank, src->dims, src->strides, dst_strides, nullptr);
  int mode;
  if (mode_override >= 0) mode = mode_override;
  else if (src->storage == ST_BF16) mode = dst_storage == ST_BF16 ? 1 : 2;
  else mode = dst_storage == ST_BF16 ? 3 : 0;
  const int block = 256, grid = grid_for(n, block);
  cudaStream_t s = c->core->stream;
  const void* sp = src->data();
  switch (mode) {
    case 0: k_copy<0><<<grid, block, 0, s>>>(it, sp, dst, n); break;
    case 1: k_copy<1><<<grid, block, 0, s>>>(it, sp, dst, n); break;
    case 2: k_copy<2><<<grid, block, 0, s>>>(it, sp, dst, n); break;
    case 3: k_copy<3><<<grid, block, 0, s>>>(it, sp, dst, n); break;
    case 4: k_copy<4><<<grid, block, 0, s>>>(it, sp, dst, n); break;
    default: k_copy<5><<<grid, block, 0, s>>>(it, sp, dst, n); break;
  }
  CG_LAUNCHED(c);
  return CG_OK;
}

int as_contiguous(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  if (x->contiguous()) {
    const_cast<cg_tensor*>(x)->rc++;
    *out = const_cast<cg_tensor*>(x);
    return CG_OK;
  }
  Hold t;
  CG_TRY(new_tensor(c, x->tag, x->storage, x->dims, x->rank, &t.t));
  CG_TRY(copy_into(c, x, t.t->data(), x->storage, t.t->strides));
  *out = t.take();
  return CG_OK;
}

int bf16_operand(cg_ctx* c, const cg_tensor* a, int64_t M, int64_t K, int64_t row_stride, int64_t col_stride, cg_tensor** keep,
                 const __nv_bfloat16** out) {
  *keep = nullptr;
  if (a->storage == ST_BF16 && col_stride == 1 && row_stride == K && ((uintptr_t)a->data() % 16) == 0) {
    *out = (const __nv_bfloat16*)a->data();
    return CG_OK;
  }
  Buffer* b = a->buf.get();
  const int64_t key[5] = {a->offset + ((int64_t)a->storage << 56), M, K, row_stride, col_stride};
  if (b->owned && b->bf16_copy && !memcmp(b->bf16_key, key, sizeof(key))) {
    *out = (const __nv_bfloat16*)b->bf16_copy->ptr;
    return CG_OK;
  }
  int64_t xd[2] = {M, K};
  Hold xa;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, xd, 2, &xa.t));
  Hold av(new_view(a));
  av.t->rank = 2;
  av.t->dims[0] = M; av.t->dims[1] = K;
  av.t->strides[0] = row_stride; av.t->strides[1] = col_stride;
  CG_TRY(copy_into(c, av.t, xa.t->data(), ST_BF16, xa.t->strides));
  *out = (const __nv_bfloat16*)xa.t->data();
  if (b->owned) {  // (memory the library does not own may be rewritten behind its back)
    b->bf16_copy = xa.t->buf;  // the copy lives as long as the buffer it was made from
    memcpy(b->bf16_key, key, sizeof(key));
  }
  *keep = xa.take();
  return CG_OK;
}

int as_contiguous_f32(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  if (x->storage != ST_BF16) return as_contiguous(c, x, out);
  Hold t;
  CG_TRY(new_tensor(c, x->tag, ST_F32, x->dims, x->rank, &t.t));
  CG_TRY(copy_into(c, x, t.t->data(), ST_F32, t.t->strides));
  *out = t.take();
  return CG_OK;
}

static bool same_shape(const cg_tensor* a, const cg_tensor* b) {
  if (a->rank != b->rank) return false;
  for (int i = 0; i < a->rank; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

template <int OP>
static int binary(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out) {
  if (!c || !a || !b || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (c->lazy && !c->lazy_busy) {
    constexpr int lb = OP == OP_ADD ? LB_ADD : OP == OP_SUB ? LB_SUB : OP == OP_MUL ? LB_MUL : OP == OP_DIV ? LB_DIV
                       : OP == OP_POW ? LB_POW : OP == OP_LT ? LB_LT : -1;
    int st = CG_OK;
    if (lb >= 0 && lazy_binary(c, lb, a, b, out, &st)) return st;
    CG_LAZY_NEED(c, a);
    CG_LAZY_NEED(c, b);
  }
  if (a->tag != b->tag) return fail(c, CG_ERR_DTYPE, "mixed dtypes in binary operation");
  if (!same_shape(a, b)) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  Hold r;
  CG_TRY(new_tensor(c, a->tag, a->tag == CG_F32 ? ST_F32 : ST_U32, a->dims, a->rank, &r.t));
  const int64_t n = r.t->numel();
  if (n) {
    cudaStream_t s = c->core->stream;
    const int block = 256;
    if (a->tag == CG_F32) {
      const bool vec = a->storage == ST_F32 && b->storage == ST_F32 && a->contiguous() && b->contiguous() &&
                       n % 4 == 0 && ((uintptr_t)a->data() % 16 == 0) && ((uintptr_t)b->data() % 16 == 0);
      if (vec) {
        k_binary_f32_vec<OP><<<grid_for(n / 4, block), block, 0, s>>>((const float4*)a->data(), (const float4*)b->data(),
                                                                     (float4*)r.t->data(), n / 4);
      } else {
        Iter it = make_iter(a->rank, a->dims, a->strides, b->strides, nullptr);
        k_binary_f32<OP><<<grid_for(n, block), block, 0, s>>>(it, a->data(), a->storage, b->data(), b->storage,
                                                            (float*)r.t->data(), n);
      }
    } else {
      Iter it = make_iter(a->rank, a->dims, a->strides, b->strides, nullptr);
      k_binary_u32<OP><<<grid_for(n, block), block, 0, s>>>(it, (const uint32_t*)a->data(), (const uint32_t*)b->data(),
                                                          (uint32_t*)r.t->data(), n);
    }
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

template <int OP>
static int unary(cg_ctx* c, const cg_tensor* x, cg_tensor** out, const char* name) {
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (OP != UN_NEG && x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, std::string("Invalid input types for ") + name);
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (OP == UN_NEG && lazy_unary_neg(c, x, out, &st)) return st;
    CG_LAZY_NEED(c, x);
  }
  Hold r;
  CG_TRY(new_tensor(c, x->tag, x->tag == CG_F32 ? ST_F32 : ST_U32, x->dims, x->rank, &r.t));
  const int64_t n = r.t->numel();
  if (n) {
    Iter it = make_iter(x->rank, x->dims, x->strides, nullptr, nullptr);
    const int block = 256, grid = grid_for(n, block);
    if (x->tag == CG_F32)
      k_unary_f32<OP><<<grid, block, 0, c->core->stream>>>(it, x->data(), x->storage, (float*)r.t->data(), n);
    else
      k_neg_u32<<<grid, block, 0, c->core->stream>>>(it, (const uint32_t*)x->data(), (uint32_t*)r.t->data(), n);
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

template <int RED>
static int reduce(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (RED != RED_ARGMAX && x->rank > 0 && lazy_reduce(c, RED == RED_MAX ? LR_MAX : LR_SUM, x, out, &st)) return st;
    CG_LAZY_NEED(c, x);
  }
  const int out_tag = RED == RED_ARGMAX ? CG_U32 : x->tag;
  const int out_st = out_tag == CG_F32 ? ST_F32 : ST_U32;
  if (x->rank == 0) {
    // rank-0 inputs pass through (shape rule of catgrad's shape-only backend)
    Hold r;
    CG_TRY(new_tensor(c, out_tag, out_st, nullptr, 0, &r.t));
    if (RED == RED_ARGMAX) CG_CUDA(c, cudaMemsetAsync(r.t->data(), 0, 4, c->core->stream));
    else CG_TRY(copy_into(c, x, r.t->data(), out_st, r.t->strides));
    *out = r.take();
    return CG_OK;
  }
  const int64_t n = x->dims[x->rank - 1];
  if (RED == RED_ARGMAX && n == 0) return fail(c, CG_ERR_SHAPE, "argmax over an empty axis");
  if (n >= (1ll << 32)) return fail(c, CG_ERR_UNSUPPORTED, "last axis too long");
  Hold xc;
  CG_TRY(as_contiguous(c, x, &xc.t));
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = 1;
  Hold r;
  CG_TRY(new_tensor(c, out_tag, out_st, od, x->rank, &r.t));
  const int64_t rows = r.t->numel();
  if (rows) {
    if (rows > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "too many rows");
    const int block = n >= 1024 ? 256 : (n >= 128 ? 128 : 32);
    if (RED == RED_ARGMAX && x->tag == CG_F32 && xc.t->storage == ST_F32 && (n & 3) == 0 && (((uintptr_t)xc.t->data()) & 15) == 0)
      k_argmax_rows_f32<<<(unsigned)rows, block, 0, c->core->stream>>>((const float*)xc.t->data(), (uint32_t*)r.t->data(), n);
    else
      k_reduce_rows<RED><<<(unsigned)rows, block, 0, c->core->stream>>>(xc.t->data(), xc.t->storage, x->tag == CG_F32,
                                                                       (uint32_t*)r.t->data(), n);
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int gemm_simt(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor* out) {
  GemmArgs g;
  const int ra = a->rank, rb = b->rank;
  g.a = a->data();
  g.b = b->data();
  g.c = out->data();
  g.sta = a->storage;
  g.stb = b->storage;
  g.M = a->dims[ra - 2];
  g.K = a->dims[ra - 1];
  g.N = b->dims[rb - 1];
  g.a_m = a->strides[ra - 2];
  g.a_k = a->strides[ra - 1];
  g.b_k = b->strides[rb - 2];
  g.b_n = b->strides[rb - 1];
  g.nb = ra - 2;
  int64_t batch = 1;
  for (int i = 0; i < ra - 2; ++i) {
    g.bd[i] = a->dims[i];
    g.ba[i] = a->strides[i];
    g.bb[i] = b->strides[i];
    batch *= a->dims[i];
  }
  if (g.M == 0 || g.N == 0 || batch == 0) return CG_OK;
  if (batch > 65535) return fail(c, CG_ERR_UNSUPPORTED, "matmul: more than 65535 batches");
  dim3 grid((unsigned)((g.N + 63) / 64), (unsigned)((g.M + 63) / 64), (unsigned)batch);
  if (grid.y > 65535) return fail(c, CG_ERR_UNSUPPORTED, "matmul: M too large for the f32 kernel");
  if (a->tag == CG_F32) k_gemm_simt<float><<<grid, 256, 0, c->core->stream>>>(g);
  else k_gemm_simt<uint32_t><<<grid, 256, 0, c->core->stream>>>(g);
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace cg

using namespace cg;

extern "C" {

int32_t cg_zeros(cg_ctx* c, const int64_t* dims, int32_t rank, int32_t dtype, cg_tensor** out) {
  if (!c || !out || (rank && !dims)) return fail(c, CG_ERR_INVALID, "bad argument");
  if (dtype != CG_F32 && dtype != CG_U32) return fail(c, CG_ERR_DTYPE, "unknown dtype");
  Hold r;
  CG_TRY(new_tensor(c, dtype, dtype == CG_F32 ? ST_F32 : ST_U32, dims, rank, &r.t));
  CG_CUDA(c, cudaMemsetAsync(r.t->data(), 0, (size_t)std::max<int64_t>(r.t->numel(), 1) * 4, c->core->stream));
  *out = r.take();
  return CG_OK;
}

static int from_vec(cg_ctx* c, int tag, const void* data, int64_t n, const int64_t* dims, int32_t rank, cg_tensor** out) {
  if (!c || !out || rank < 0 || rank > CG_MAX_RANK || (rank && !dims) || (n && !data)) return fail(c, CG_ERR_INVALID, "bad argument");
  int64_t want = 1;
  for (int i = 0; i < rank; ++i) want *= dims[i];
  if (want != n) return fail(c, CG_ERR_SHAPE, "ShapeError");
  const bool as_bf16 = tag == CG_F32 && c->precision == CG_PREC_BF16 && rank >= 2;
  Hold r;
  CG_TRY(new_tensor(c, tag, tag == CG_F32 ? ST_F32 : ST_U32, dims, rank, &r.t));
  if (n) {
    // pageable source: the copy is staged by the driver and the call returns once the
    // source has been read, so the caller may free `data` at once
    CG_CUDA(c, cudaMemcpyAsync(r.t->data(), data, (size_t)n * 4, cudaMemcpyHostToDevice, c->core->stream));
  }
  if (as_bf16) {
    cg_tensor* b = nullptr;
    CG_TRY(cg_to_bf16(c, r.t, &b));
    *out = b;
    return CG_OK;
  }
  if (n == 1) {  // a literal: its value stays known on the host
    r.t->has_scalar = true;
    memcpy(&r.t->scalar_bits, data, 4);
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_ndarray_from_vec_f32(cg_ctx* c, const float* d, int64_t n, const int64_t* dims, int32_t rank, cg_tensor** out) {
  return from_vec(c, CG_F32, d, n, dims, rank, out);
}
int32_t cg_ndarray_from_vec_u32(cg_ctx* c, const uint32_t* d, int64_t n, const int64_t* dims, int32_t rank, cg_tensor** out) {
  return from_vec(c, CG_U32, d, n, dims, rank, out);
}

int32_t cg_to_bf16(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  CG_LAZY_NEED(c, x);
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "bf16 storage is for F32-tagged tensors");
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, x->dims, x->rank, &r.t));
  CG_TRY(copy_into(c, x, r.t->data(), ST_BF16, r.t->strides));
  *out = r.take();
  return CG_OK;
}

int32_t cg_to_f32(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  CG_LAZY_NEED(c, x);
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "not an F32-tagged tensor");
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
  CG_TRY(copy_into(c, x, r.t->data(), ST_F32, r.t->strides));
  *out = r.take();
  return CG_OK;
}

int32_t cg_cast(cg_ctx* c, const cg_tensor* x, int32_t dtype, cg_tensor** out) {
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (dtype != CG_F32 && dtype != CG_U32) return fail(c, CG_ERR_DTYPE, "unknown dtype");
  if (x->tag == dtype) {
    const_cast<cg_tensor*>(x)->rc++;
    *out = const_cast<cg_tensor*>(x);
    return CG_OK;
  }
  if (x->has_scalar && !x->node && x->numel() == 1) {
    // a literal whose value is known on the host (e.g. the element count an rmsnorm divides by,
    // cast from a Nat): convert it here and upload the result, no kernel
    uint32_t bits;
    if (dtype == CG_F32) {
      const float v = (float)x->scalar_bits;
      memcpy(&bits, &v, 4);
    } else {
      float v;
      memcpy(&v, &x->scalar_bits, 4);
      bits = !(v == v) ? 0u : v <= 0.f ? 0u : v >= 4294967296.f ? 0xFFFFFFFFu : (uint32_t)v;  // Rust's `as`: saturating, NaN -> 0
    }
    return from_vec(c, dtype, &bits, 1, x->dims, x->rank, out);
  }
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (lazy_cast(c, x, dtype, out, &st)) return st;
    CG_LAZY_NEED(c, x);
  }
  Hold src;
  CG_TRY(as_contiguous_f32(c, x, &src.t));  // also widens bf16
  Hold r;
  CG_TRY(new_tensor(c, dtype, dtype == CG_F32 ? ST_F32 : ST_U32, x->dims, x->rank, &r.t));
  CG_TRY(copy_into(c, src.t, r.t->data(), r.t->storage, r.t->strides, dtype == CG_U32 ? 4 : 5));
  if (x->has_scalar) {
    // the literal's value follows it through the cast (f32 -> u32 saturates, NaN -> 0, as `as` does)
    r.t->has_scalar = true;
    if (dtype == CG_F32) {
      const float v = (float)x->scalar_bits;
      memcpy(&r.t->scalar_bits, &v, 4);
    } else {
      float v;
      memcpy(&v, &x->scalar_bits, 4);
      r.t->scalar_bits = !(v == v) ? 0u : v <= 0.f ? 0u : v >= 4294967296.f ? 0xFFFFFFFFu : (uint32_t)v;
    }
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_add(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_ADD>(c, a, b, o); }
int32_t cg_sub(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_SUB>(c, a, b, o); }
int32_t cg_mul(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_MUL>(c, a, b, o); }
int32_t cg_div(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_DIV>(c, a, b, o); }
int32_t cg_pow(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_POW>(c, a, b, o); }
int32_t cg_lt(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_LT>(c, a, b, o); }
int32_t cg_eq(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** o) { return binary<OP_EQ>(c, a, b, o); }
int32_t cg_sin(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return unary<UN_SIN>(c, x, o, "sin"); }
int32_t cg_cos(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return unary<UN_COS>(c, x, o, "cos"); }
int32_t cg_neg(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return unary<UN_NEG>(c, x, o, "neg"); }
int32_t cg_max(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return reduce<RED_MAX>(c, x, o); }
int32_t cg_sum(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return reduce<RED_SUM>(c, x, o); }
int32_t cg_argmax(cg_ctx* c, const cg_tensor* x, cg_tensor** o) { return reduce<RED_ARGMAX>(c, x, o); }

int32_t cg_topk(cg_ctx* c, const cg_tensor* x, int64_t k, cg_tensor** values, cg_tensor** indices) {
  CG_LAZY_NEED(c, x);
  if (!c || !x || !values || !indices) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "Unsupported type for topk");
  if (x->rank == 0) return fail(c, CG_ERR_SHAPE, "topk of a rank-0 tensor");
  const int64_t n = x->dims[x->rank - 1];
  if (k < 0 || k > n) return fail(c, CG_ERR_SHAPE, "topk: k exceeds the last dimension");
  if (n >= 0xFFFFFFFFll) return fail(c, CG_ERR_UNSUPPORTED, "last axis too long");
  Hold xc;
  CG_TRY(as_contiguous_f32(c, x, &xc.t));
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = k;
  Hold v, ix;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, od, x->rank, &v.t));
  CG_TRY(new_tensor(c, CG_U32, ST_U32, od, x->rank, &ix.t));
  const int64_t rows = n ? x->numel() / n : 0;
  if (rows && k) {
    if (rows > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "too many rows");
    const int block = n >= 1024 ? 256 : (n >= 128 ? 128 : 32);
    k_topk_rows<<<(unsigned)rows, block, 0, c->core->stream>>>((const float*)xc.t->data(), (float*)v.t->data(),
                                                              (uint32_t*)ix.t->data(), n, k);
    CG_LAUNCHED(c);
  }
  *values = v.take();
  *indices = ix.take();
  return CG_OK;
}

int32_t cg_compare(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, int32_t* equal) {
  CG_LAZY_NEED(c, a);
  CG_LAZY_NEED(c, b);
  if (!c || !a || !b || !equal) return fail(c, CG_ERR_INVALID, "null argument");
  if (a->tag != b->tag) return fail(c, CG_ERR_DTYPE, "mixed dtypes in compare");
  *equal = 0;
  if (!same_shape(a, b)) return CG_OK;
  const int64_t n = a->numel();
  int32_t host = 1;
  if (n) {
    int64_t one = 1;
    Hold flag;
    CG_TRY(new_tensor(c, CG_U32, ST_U32, &one, 1, &flag.t));
    CG_CUDA(c, cudaMemcpyAsync(flag.t->data(), &host, 4, cudaMemcpyHostToDevice, c->core->stream));
    Iter it = make_iter(a->rank, a->dims, a->strides, b->strides, nullptr);
    k_compare<<<grid_for(n, 256), 256, 0, c->core->stream>>>(it, a->data(), a->storage, b->data(), b->storage,
                                                            a->tag == CG_F32, n, (int32_t*)flag.t->data());
    CG_LAUNCHED(c);
    CG_CUDA(c, cudaMemcpyAsync(&host, flag.t->data(), 4, cudaMemcpyDeviceToHost, c->core->stream));
    CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  }
  *equal = host;
  return CG_OK;
}

int32_t cg_concat(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, int32_t dim, cg_tensor** out) {
  if (!c || !a || !b || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (lazy_concat(c, a, b, dim, out, &st)) return st;
    CG_LAZY_NEED(c, a);
    CG_LAZY_NEED(c, b);
  }
  if (a->tag != b->tag) return fail(c, CG_ERR_DTYPE, "Incompatible types for concatenation");
  if (a->rank != b->rank || dim < 0 || dim >= a->rank) return fail(c, CG_ERR_SHAPE, "concat: rank or axis mismatch");
  for (int i = 0; i < a->rank; ++i)
    if (i != dim && a->dims[i] != b->dims[i]) return fail(c, CG_ERR_SHAPE, "concat: shapes differ off the axis");
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < a->rank; ++i) od[i] = a->dims[i];
  od[dim] += b->dims[dim];
  const int st = (a->storage == ST_BF16 && b->storage == ST_BF16) ? ST_BF16 : (a->tag == CG_F32 ? ST_F32 : ST_U32);
  Hold r;
  CG_TRY(new_tensor(c, a->tag, st, od, a->rank, &r.t));
  CG_TRY(copy_into(c, a, r.t->data(), st, r.t->strides));
  void* second = (char*)r.t->data() + (size_t)(a->dims[dim] * r.t->strides[dim]) * storage_bytes(st);
  CG_TRY(copy_into(c, b, second, st, r.t->strides));
  *out = r.take();
  return CG_OK;
}

int32_t cg_index(cg_ctx* c, const cg_tensor* x, int32_t dim, const cg_tensor* indices, cg_tensor** out) {
  CG_LAZY_NEED(c, x);
  CG_LAZY_NEED(c, indices);
  if (!c || !x || !indices || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (indices->tag != CG_U32) return fail(c, CG_ERR_DTYPE, "Invalid input types for indexing");
  if (dim < 0 || dim >= x->rank) return fail(c, CG_ERR_SHAPE, "index: axis out of range");
  Hold xc, ic;
  CG_TRY(as_contiguous(c, x, &xc.t));
  CG_TRY(as_contiguous(c, indices, &ic.t));
  const int64_t ni = indices->numel();
  int64_t od[CG_MAX_RANK], outer = 1, inner = 1;
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[dim] = ni;
  for (int i = 0; i < dim; ++i) outer *= x->dims[i];
  for (int i = dim + 1; i < x->rank; ++i) inner *= x->dims[i];
  Hold r;
  CG_TRY(new_tensor(c, x->tag, x->storage, od, x->rank, &r.t));
  const int64_t n = r.t->numel();
  if (n) {
    if (x->dims[dim] == 0) return fail(c, CG_ERR_INDEX, "index out of bounds");
    const int64_t row_bytes = inner * (int64_t)storage_bytes(x->storage);
    const bool rows_vec = row_bytes >= 256 && row_bytes % 16 == 0 && ((((uintptr_t)xc.t->data()) | ((uintptr_t)r.t->data())) & 15) == 0;
    if (rows_vec) {
      const int64_t rows = outer * ni;
      const int block = row_bytes / 16 >= 256 ? 256 : (row_bytes / 16 >= 64 ? 64 : 32);
      k_index_rows<<<(unsigned)std::min<int64_t>(rows, 148 * 64), block, 0, c->core->stream>>>(
          (const uint4*)xc.t->data(), (const uint32_t*)ic.t->data(), (uint4*)r.t->data(), x->dims[dim], ni, rows, row_bytes / 16,
          c->core->dev_err);
    } else if (x->storage == ST_BF16)
      k_index16<<<grid_for(n, 256), 256, 0, c->core->stream>>>((const uint16_t*)xc.t->data(), (const uint32_t*)ic.t->data(),
                                                              (uint16_t*)r.t->data(), outer, x->dims[dim], ni, inner,
                                                              c->core->dev_err);
    else
      k_index<<<grid_for(n, 256), 256, 0, c->core->stream>>>((const uint32_t*)xc.t->data(), (const uint32_t*)ic.t->data(),
                                                            (uint32_t*)r.t->data(), outer, x->dims[dim], ni, inner,
                                                            c->core->dev_err);
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_arange(cg_ctx* c, int64_t end, cg_tensor** out) {
  if (!c || !out || end < 0) return fail(c, CG_ERR_INVALID, "bad argument");
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (lazy_arange(c, end, out, &st)) return st;
  }
  int64_t n = (int64_t)ceilf((float)end);
  Hold r;
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &r.t));
  if (n) {
    k_arange<<<grid_for(n, 256), 256, 0, c->core->stream>>>((uint32_t*)r.t->data(), n);
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

static int to_vec(cg_ctx* c, int tag, const cg_tensor* x, void* dst, int64_t n) {
  if (!c || !x || (!dst && n)) return fail(c, CG_ERR_INVALID, "null argument");
  CG_LAZY_NEED(c, x);
  if (x->tag != tag) return fail(c, CG_ERR_DTYPE, "to_vec: dtype tag differs");
  if (n != x->numel()) return fail(c, CG_ERR_SHAPE, "to_vec: element count differs");
  Hold src;
  CG_TRY(as_contiguous_f32(c, x, &src.t));
  if (n) CG_CUDA(c, cudaMemcpyAsync(dst, src.t->data(), (size_t)n * 4, cudaMemcpyDeviceToHost, c->core->stream));
  return cg_sync(c);
}
int32_t cg_to_vec_f32(cg_ctx* c, const cg_tensor* x, float* dst, int64_t n) { return to_vec(c, CG_F32, x, dst, n); }
int32_t cg_to_vec_u32(cg_ctx* c, const cg_tensor* x, uint32_t* dst, int64_t n) { return to_vec(c, CG_U32, x, dst, n); }

int32_t cg_matmul(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out) {
  if (!c || !a || !b || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (c->lazy && !c->lazy_busy) {
    int st = CG_OK;
    if (lazy_matmul(c, a, b, out, &st)) return st;
    CG_LAZY_NEED(c, a);
    CG_LAZY_NEED(c, b);
  }
  if (a->tag != b->tag) return fail(c, CG_ERR_DTYPE, "mixed dtypes in matmul");
  const int ra = a->rank, rb = b->rank;
  if (ra < 2) return fail(c, CG_ERR_SHAPE, "batched_matmul: lhs must be at least rank 2");
  if (rb < 2) return fail(c, CG_ERR_SHAPE, "batched_matmul: rhs must be at least rank 2");
  if (a->dims[ra - 1] != b->dims[rb - 2]) return fail(c, CG_ERR_SHAPE, "batched_matmul: incompatible matrix dimensions");
  if (ra != rb) return fail(c, CG_ERR_SHAPE, "batched_matmul: batch dimensions must match");
  for (int i = 0; i < ra - 2; ++i)
    if (a->dims[i] != b->dims[i]) return fail(c, CG_ERR_SHAPE, "batched_matmul: batch dimensions must match");
  int64_t od[CG_MAX_RANK];
  int64_t batch = 1;
  for (int i = 0; i < ra - 2; ++i) { od[i] = a->dims[i]; batch *= a->dims[i]; }
  const int64_t M = a->dims[ra - 2], K = a->dims[ra - 1], N = b->dims[rb - 1];
  od[ra - 2] = M;
  od[ra - 1] = N;
  Hold r;
  CG_TRY(new_tensor(c, a->tag, a->tag == CG_F32 ? ST_F32 : ST_U32, od, ra, &r.t));
  if (r.t->numel() == 0) { *out = r.take(); return CG_OK; }
  if (K == 0) {
    CG_CUDA(c, cudaMemsetAsync(r.t->data(), 0, (size_t)r.t->numel() * 4, c->core->stream));
    *out = r.take();
    return CG_OK;
  }
  // A weight stored bf16 and seen through transpose (k unit-stride, rows K apart or more):
  // round the activations to bf16 and use the tensor-core pipeline.
  const bool tc = c->opt_gemm == 0 && a->tag == CG_F32 && batch == 1 && b->storage == ST_BF16 &&
                  b->strides[rb - 2] == 1 && b->strides[rb - 1] >= K && b->strides[rb - 1] % 8 == 0 && K % 8 == 0 &&
                  ((uintptr_t)b->data() % 16 == 0);
  if (tc) {
    // a as a bf16 [M, K] matrix (shared with the other GEMMs that read the same activations)
    Hold xa;
    const __nv_bfloat16* xp;
    CG_TRY(bf16_operand(c, a, M, K, a->strides[ra - 2], a->strides[ra - 1], &xa.t, &xp));
    CG_TRY(gemm_tc(c, xp, K, (const __nv_bfloat16*)b->data(), b->strides[rb - 1],
                   r.t->data(), N, nullptr, M, N, K, 0, 0, nullptr));
  } else {
    CG_TRY(gemm_simt(c, a, b, r.t));
  }
  *out = r.take();
  return CG_OK;
}

}  // extern "C"
