// attn_decode.cu — one kernel for the attention block of a decode step.
//
// For one new token per row it does, per (row, kv head), what the reference spreads over
// reshape/transpose, optional per-head RMSNorm (catgrad-llm/src/models/qwen3.rs:187-217),
// apply_rope_embedding (catgrad-llm/src/helpers.rs:202-221), repeat_kv (helpers.rs:147-161),
// the masked softmax(q k^T / sqrt(d)) v of catgrad-llm/src/models/llama.rs:97-108 and the
// cache append of catgrad-llm/src/legacy/models/utils.rs:210-228:
//
//   1. request this CTA's slice of cached keys and values (16-byte cp.async, coalesced)
//      before anything else, then, while they fly, split the f32 qkv row, normalise / rotate
//      q and the new k, round them to bf16 (the cache precision) and append k, v to the cache;
//   2. the query heads that share the kv head are the rows of one 16-row MMA tile, so
//      q k^T and p v for 32 keys are a few mma.sync instructions per warp instead of
//      thousands of scalar FMAs; online softmax per head;
//   3. the slices of one (row, kv head) form a thread-block cluster: each leaves its partial
//      (max, sum, weighted values) in shared memory and, after one cluster barrier, the
//      partials are merged over distributed shared memory into the bf16 output that the
//      output projection reads.  No scratch in HBM, no second kernel.
//
// The whole block is latency-bound (a few MB per layer), so the design minimises dependent
// round trips and instruction count rather than bytes.
#include <algorithm>

#include "attn_decode.cuh"
#include "kernels.h"
#include "mma.cuh"

namespace cg {

namespace {

constexpr int MAX_REP = ATTN_MAX_REP;

// one CTA per item; the slices of one (row, kv head) are one thread-block cluster
struct KernelEnv {
  __device__ __forceinline__ int tid() const { return threadIdx.x; }
  __device__ __forceinline__ void sync_cta() const { __syncthreads(); }
  __device__ __forceinline__ void sync_group() const {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  __device__ __forceinline__ uint32_t cluster_rank(int s) const { return (uint32_t)s; }
  // one item per CTA: partials are pushed into the finishing CTA's landing area
  static constexpr bool kPush = true;
  float* land;
  __device__ __forceinline__ float* landing() const { return land; }
  // the projected row, and the position when it lives on the device, belong to the stream order
  const AttnDecArgs* args;
  __device__ __forceinline__ int64_t settle(int64_t) const {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    return args->pos_dev ? *(const volatile int64_t*)args->pos_dev : args->pos0;
  }
};

template <int D>
__global__ void __launch_bounds__(128) k_attn_dec(AttnDecArgs a, float scale) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ __align__(16) uint8_t smem[];
  KernelEnv env;
  env.args = &a;
  env.land = (float*)(smem + attn_dec_smem_bytes<D>());
  // Before the dependency wait: the first tiles of cached keys and values can be on the way
  // while the projection GEMM still runs.  What makes that sound: every writer of the device-side
  // position (the one-thread state kernel, in plain stream order; the arg-max kernel, after its
  // own dependency wait) stores a value v only after every kernel that wrote cache rows below v
  // has completed, so whatever value is visible here, the rows below it are complete.  The value
  // may be a step old; it is re-read after the wait and a changed value repeats the request.
  int64_t pos_early = a.pos_dev ? *(const volatile int64_t*)a.pos_dev : a.pos0;
  pos_early = pos_early < 0 ? 0 : (pos_early >= a.Tmax ? a.Tmax - 1 : pos_early);
  attn_dec_item<D>(a, scale, (int)blockIdx.x, (int64_t)blockIdx.y, (int)blockIdx.z, pos_early, smem, env);
}

template <int D>
int launch(cg_ctx* c, const AttnDecArgs& args) {
  constexpr int LD = D + 8;
  constexpr int KT = D > 128 ? 16 : 32;
  AttnDecArgs a = args;
  // The push form of the slice merge needs a landing area nothing else uses; it is taken only
  // where that does not cost a resident CTA per SM (head size 128 would drop from three to two,
  // which measured 1 % slower per step on the mixture-of-experts shape).
  const int rep = a.nh / a.nkv;
  const int blocks = a.splits * ((rep * D + 128 * a.splits - 1) / (128 * a.splits));
  const size_t land = (size_t)(8 * MAX_REP * 2 + blocks * 128) * 4;
  auto per_sm = [](size_t bytes) { return (227 * 1024) / (bytes + 1024); };
  a.push_merge = a.splits > 1 && a.splits <= 8 && land <= attn_dec_landing_bytes() &&
                 per_sm(attn_dec_smem_bytes<D>() + land) == per_sm(attn_dec_smem_bytes<D>());
  const size_t smem = attn_dec_smem_bytes<D>() + (a.push_merge ? land : 0);
  static_assert(attn_dec_smem_bytes<D>() == (size_t)(16 * LD + 8 * KT * LD) * 2 + (size_t)(2 * D + 8 * MAX_REP + 16) * 4, "layout");
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured && attn_dec_smem_bytes<D>() + attn_dec_landing_bytes() > 48 * 1024) {
    CG_CUDA(c, cudaFuncSetAttribute(k_attn_dec<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(attn_dec_smem_bytes<D>() + attn_dec_landing_bytes())));
    configured = true;
  }
  static PerDeviceFlag wide_on;
  bool& wide = wide_on.at(c->core->device);
  if (!wide && a.splits > 8) {
    CG_CUDA(c, cudaFuncSetAttribute(k_attn_dec<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    wide = true;
  }
  dim3 grid((unsigned)a.nkv, (unsigned)a.B, (unsigned)a.splits);
  CG_CUDA(c, launch_kernel(c, k_attn_dec<D>, grid, dim3(128), smem, a.splits, a, 1.0f / sqrtf((float)D)));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

// context slices per (row, kv head): a power of two up to 8 (one portable cluster), about
// 128 keys per slice at full context
int attn_dec_splits(int64_t Tmax, int64_t pairs, int d) {
  int s = 1;
  while (s < 8 && (int64_t)s * 128 < Tmax) s *= 2;
  // (head size 256 once had 32-key tiles: 143 KB per CTA, one CTA per SM, and clusters of 8 such
  // CTAs did not all fit at once -- 128 CTAs took two waves; with 16-key tiles three CTAs share
  // an SM)
  (void)d;
  // (16 slices -- a cluster size this GPU supports beyond the portable 8 -- were measured for
  // few (row, kv head) pairs with long contexts and were slower: 2.92 -> 3.15 ms per step on
  // the 256-wide heads of the Gemma shape.)
  // many (row, kv head) pairs: fewer, longer slices, so that the fixed cost of a CTA (query
  // preparation, merges) is spread over more keys; keep about four waves of CTAs
  while (s > 1 && pairs * s > 4 * 3 * 148 && (int64_t)(s / 2) * 1024 >= Tmax / 4) s /= 2;
  return s;
}

int k_launch_attn_dec(cg_ctx* c, const AttnDecArgs& a) {
  if (a.nkv <= 0 || a.nh % a.nkv || a.nh / a.nkv > MAX_REP)
    return fail(c, CG_ERR_UNSUPPORTED, "attention decode: query heads per kv head must be 1..8");
  if (a.d != 64 && a.d != 128 && a.d != 256) return fail(c, CG_ERR_UNSUPPORTED, "attention: head_dim must be 64, 128 or 256");
  if (a.B > 65535) return fail(c, CG_ERR_UNSUPPORTED, "attention: too many rows");
  if (!a.pos_dev && a.pos0 >= a.Tmax) return fail(c, CG_ERR_SHAPE, "attention: KV cache capacity exceeded");
  if (a.B == 0) return CG_OK;
  switch (a.d) {
    case 64: return launch<64>(c, a);
    case 128: return launch<128>(c, a);
    default: return launch<256>(c, a);
  }
}

}  // namespace cg
