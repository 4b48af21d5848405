// noalloc.cu — row-wise arg-max for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a result: code
// running while a CUDA graph is being captured on another stream of the process, plugins that
// are handed a fixed memory budget by their embedding application, and real-time loops where an
// allocation (which may synchronise the device) is not acceptable.  The regular arg-max path
// takes its merge slots (one 64-bit word per row) from the context's allocator; this variant
// keeps them in a file-scope device array instead, so the call touches nothing but the caller's
// input and output buffers and that array.
//
// Limits and rules:
//   * at most CG_NOALLOC_MAX_ROWS rows per call (the array is 8 bytes per row, 32 KiB, and is
//     held by every GPU that loads the library until the process exits);
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress with
//     that device current) and caches it; make that first call outside of any stream capture;
//   * every call shares the one array: two calls that overlap on the GPU (different streams)
//     race on it.  Calls on one stream are ordered and safe.  The slots a call uses are zeroed
//     at its start, whatever an earlier call left behind.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/catgrad_cuda.h"

namespace {

// merge slots: (total-order key << 32 | index), folded with a 64-bit atomic max
__device__ __align__(256) unsigned long long g_noalloc_best[CG_NOALLOC_MAX_ROWS];

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
unsigned long long* g_slots[MAX_DEVICES] = {nullptr};  // device address of g_noalloc_best, per device

__global__ void k_na_part(const float* x, int64_t n, unsigned long long* best) {
  __shared__ unsigned long long sh[32];
  const int64_t row = blockIdx.y;
  const int64_t span = (n + gridDim.x - 1) / gridDim.x;
  const int64_t i0 = blockIdx.x * span, i1 = min(n, i0 + span);
  unsigned long long m = 0;
  for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    const uint32_t bits = __float_as_uint(x[row * n + i]);
    const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // f32::total_cmp order
    const unsigned long long q = ((unsigned long long)key << 32) | (uint32_t)i;  // ties -> last index
    m = q > m ? q : m;
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int o = 16; o; o >>= 1) {
    const unsigned long long w = __shfl_xor_sync(0xffffffffu, m, o);
    m = w > m ? w : m;
  }
  if (lane == 0) sh[wid] = m;
  __syncthreads();
  if (wid == 0) {
    m = lane < nw ? sh[lane] : 0ull;
    for (int o = 16; o; o >>= 1) {
      const unsigned long long w = __shfl_xor_sync(0xffffffffu, m, o);
      m = w > m ? w : m;
    }
    if (lane == 0 && i0 < i1) atomicMax(best + row, m);
  }
}

__global__ void k_na_finish(const unsigned long long* best, int64_t rows, uint32_t* out) {
  const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (r < rows) out[r] = (uint32_t)(best[r] & 0xFFFFFFFFull);
}

int fail(char* err, int64_t cap, int code, const char* msg) {
  if (err && cap > 0) snprintf(err, (size_t)cap, "%s", msg);
  return code;
}

}  // namespace

extern "C" int32_t cg_argmax_rows_noalloc(void* stream, const float* logits, int64_t rows, int64_t n, uint32_t* out,
                                          char* err, int64_t err_cap) {
  if (err && err_cap > 0) err[0] = 0;
  if (rows < 0 || n < 0 || (rows && (!logits || !out))) return fail(err, err_cap, CG_ERR_INVALID, "null pointer or negative size");
  if (rows > CG_NOALLOC_MAX_ROWS) {
    char msg[160];
    snprintf(msg, sizeof msg, "cg_argmax_rows_noalloc: %lld rows exceed the fixed scratch of %d rows", (long long)rows,
             CG_NOALLOC_MAX_ROWS);
    return fail(err, err_cap, CG_ERR_INVALID, msg);
  }
  if (n == 0 && rows) return fail(err, err_cap, CG_ERR_SHAPE, "argmax over an empty axis");
  if (n >= (1ll << 32)) return fail(err, err_cap, CG_ERR_UNSUPPORTED, "last axis too long");
  if (rows == 0) return CG_OK;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return fail(err, err_cap, CG_ERR_CUDA, "no current CUDA device");
  unsigned long long* slots = nullptr;
  {
    // set-up, once per device, with that device current: the array's name is only a host-side
    // stand-in, kernels need its device address
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_slots[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_best);
      if (e != cudaSuccess) return fail(err, err_cap, CG_ERR_CUDA, cudaGetErrorString(e));
      g_slots[dev] = (unsigned long long*)p;
    }
    slots = g_slots[dev];
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(slots, 0, (size_t)rows * 8, s);  // the array keeps the last call's contents
  if (e != cudaSuccess) return fail(err, err_cap, CG_ERR_CUDA, cudaGetErrorString(e));
  const unsigned chunks = (unsigned)(n >= 65536 ? 64 : n >= 1024 ? n / 1024 : 1);
  // grid.y is limited to 65535 rows, far above the scratch limit
  k_na_part<<<dim3(chunks, (unsigned)rows), 256, 0, s>>>(logits, n, slots);
  k_na_finish<<<(unsigned)((rows + 127) / 128), 128, 0, s>>>(slots, rows, out);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(err, err_cap, CG_ERR_CUDA, cudaGetErrorString(e));
  return CG_OK;
}
