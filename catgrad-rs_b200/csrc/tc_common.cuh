// tc_common.cuh — inline PTX shared by the tensor-core GEMM kernels: mbarriers with bounded
// waits, TMA tile loads, tcgen05 descriptors / MMA / TMEM loads, cluster barriers and
// distributed-shared-memory loads.
#pragma once

#include <cuda.h>

#include "runtime.h"

namespace cg {
namespace tc {

constexpr int BM = 128;       // W rows per CTA (MMA M)
constexpr int BK = 64;        // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// The context's device error block: word 0 is the error code (DevErr), the 64-bit word at byte
// offset 8 is the limit of every bounded wait in nanoseconds (set by the host; 0 reads as 1 s).
__device__ __forceinline__ uint64_t wait_limit_ns(const int32_t* err) {
  const uint64_t v = *(const volatile uint64_t*)(err + 2);
  return v ? v : 1000000000ull;
}
// Bounded wait on an mbarrier phase.  Returns false once the limit has passed (raising *err),
// once another wait of this CTA has already given up, or once any kernel of the context has
// reported a timeout: after the first expiry every later wait gives up at its first slow-path
// check, so a lost producer costs one limit in total instead of one per wait.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort, int32_t* err) {
  uint32_t done = 0;
  uint64_t t0 = 0, limit = 0;
  for (uint32_t it = 0;; ++it) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 0x3FF) == 0x3FF) {
      if (*cta_abort) return false;
      if (*(volatile int32_t*)err == DEV_TIMEOUT) break;
      uint64_t now = globaltimer();
      if (t0 == 0) { t0 = now; limit = wait_limit_ns(err); }
      else if (now - t0 > limit) break;
    }
  }
  *cta_abort = 1;
  *err = DEV_TIMEOUT;
  return false;
}

__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_bar), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// Bounded wait on an mbarrier other CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* cta_abort, int32_t* err) {
  uint32_t done = 0;
  uint64_t t0 = 0, limit = 0;
  for (uint32_t it = 0;; ++it) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 0x3FF) == 0x3FF) {
      if (*cta_abort) return false;
      if (*(volatile int32_t*)err == DEV_TIMEOUT) break;
      uint64_t now = globaltimer();
      if (t0 == 0) { t0 = now; limit = wait_limit_ns(err); }
      else if (now - t0 > limit) break;
    }
  }
  *cta_abort = 1;
  *err = DEV_TIMEOUT;
  return false;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor for a k-major, 128B-swizzled tile whose rows are 128
// bytes: 8-row groups are 1024 bytes apart (SBO), LBO is unused for swizzled k-major.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (ignored)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // descriptor version for this architecture
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, both operands k-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Sum over the `n` (<= 16) CTAs of a cluster of the float at the same shared-memory offset, in
// rank order.  All loads are issued before the first add, so their latencies overlap (a loop
// of "load, add" would pay one distributed-shared-memory round trip per rank).
__device__ __forceinline__ float sum_cluster_f32(uint32_t local_addr, int n) {
  float v[16];
#pragma unroll
  for (int s = 0; s < 16; ++s) v[s] = s < n ? ld_cluster_f32(local_addr, (uint32_t)s) : 0.f;
  float acc = 0.f;
#pragma unroll
  for (int s = 0; s < 16; ++s) acc += v[s];  // adding the zeros of absent ranks changes nothing
  return acc;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld:
// boxes of [box_rows, 64] elements, 128-byte swizzle, zero fill outside the matrix.
inline int make_map(cg_ctx* c, CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  if (!c->encode_tiled) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return fail(c, CG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    c->encode_tiled = fn;
  }
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = ((EncodeTiledFn)c->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim,
                                                gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, CG_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return CG_OK;
}

}  // namespace tc
}  // namespace cg
