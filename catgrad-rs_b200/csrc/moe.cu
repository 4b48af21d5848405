// moe.cu — the mixture-of-experts feed-forward block of catgrad-llm/src/models/qwen3.rs:64-133
// for the fused decoder.
//
// The reference gathers, for every token and every one of its top-k slots, a whole expert
// matrix (index along the expert axis) and applies it with a batched matmul.  Here the
// (token, slot) pairs are grouped by expert instead, so every expert matrix is streamed from
// HBM once per layer however many tokens chose it:
//
//   k_moe_route    per token: RMSNorm, router logits (f32), softmax, top-k (ties -> lower
//                  expert id, as the reference's topk), optional renormalisation
//   k_moe_plan     histogram of the pairs over the experts this rank owns, offsets, the tile
//                  list of the grouped GEMMs, and each pair's row in the grouped order
//   k_moe_gather   bf16 activation rows copied into grouped order
//   k_moe_gemm     grouped tcgen05 GEMM over the tile list: gate and up projections share a
//                  CTA (two TMEM accumulators) with act(gate) * up as the epilogue; the same
//                  kernel without the pairing does the down projection
//   k_moe_combine  per token: sum over its slots (in slot order) of weight * expert output,
//                  added to the residual stream
//
// Expert parallelism: a rank that owns experts [e_lo, e_hi) plans only the pairs routed to
// them; pairs of other ranks contribute nothing and the per-rank partial sums are added by
// the caller's all-reduce.
#include <algorithm>

#include "act.cuh"
#include "kernels.h"
#include "peer.cuh"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

__device__ __forceinline__ float block_sum_f(float v, float* sh) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  v = lane < nw ? sh[lane] : 0.f;
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  return v;  // every thread of every warp holds the total
}

// Sum of the k values held one per lane (lane r holds value r, k <= 32) in the order of the
// reference's reduction: ndarray folds a contiguous lane with eight interleaved partial sums,
// combines them as ((p0+p4)+(p1+p5))+((p2+p6)+(p3+p7)) and adds the tail in order (the checker's
// lane_sum).  Called by all 32 lanes; every lane gets the same bits.
__device__ __forceinline__ float sum_in_reference_order(float mine, int k) {
  float p[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int i = 0;
  for (; i + 8 <= k; i += 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = p[j] + __shfl_sync(0xffffffffu, mine, i + j);
  }
  float acc = 0.f;
  acc = acc + (p[0] + p[4]);
  acc = acc + (p[1] + p[5]);
  acc = acc + (p[2] + p[6]);
  acc = acc + (p[3] + p[7]);
  for (; i < k; ++i) acc = acc + __shfl_sync(0xffffffffu, mine, i);
  return acc;
}

// One block per token.  Shared memory: xs[H] normalised row, pr[E] router probabilities.
__global__ void k_moe_route(const float* x, const float* gamma, float eps, int plus_one, const float* wr, int H, int E, int k,
                            int norm_topk, __nv_bfloat16* xn, uint32_t* ids, float* wts) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float sm[];
  __shared__ float red[32];
  float* xs = sm;
  float* pr = sm + H;
  const int64_t m = blockIdx.x;
  const float* row = x + m * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ss += row[i] * row[i];
  ss = block_sum_f(ss, red);
  const float rms = sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    // without norm weights the rows are taken as they are (the caller normalised them)
    const float v = gamma ? row[i] / rms * (plus_one ? 1.f + gamma[i] : gamma[i]) : row[i];
    xs[i] = v;
    xn[m * H + i] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  // router logits: one warp per expert, lanes stride the hidden axis
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int e = wid; e < E; e += nw) {
    const float* w = wr + (int64_t)e * H;
    float acc = 0.f;
    for (int i = lane; i < H; i += 32) acc += xs[i] * w[i];
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) pr[e] = acc;
  }
  __syncthreads();
  if (wid != 0) return;
  // softmax over the experts (catgrad/src/stdlib/nn/mod.rs:104-126: subtract the max, exp, divide by the sum)
  float mx = -3.4028234663852886e38f;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, pr[e]);
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(pr[e] - mx);
    pr[e] = v;
    sum += v;
  }
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) pr[e] = pr[e] / sum;
  __syncwarp();
  // top-k by k rounds of arg-max; ties go to the lower expert id
  float chosen = 0.f, total = 0.f;
  uint32_t chosen_id = 0;
  for (int r = 0; r < k; ++r) {
    unsigned long long best = 0;
    for (int e = lane; e < E; e += 32) {
      const float v = pr[e];
      if (v < 0.f) continue;  // taken (probabilities are never negative)
      const unsigned long long q = ((unsigned long long)__float_as_uint(v) << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)e);
      best = q > best ? q : best;
    }
    for (int o = 16; o; o >>= 1) {
      const unsigned long long w = __shfl_xor_sync(0xffffffffu, best, o);
      best = w > best ? w : best;
    }
    const uint32_t e = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull);
    const float v = __uint_as_float((uint32_t)(best >> 32));
    if (lane == r) { chosen = v; chosen_id = e; }  // k <= 32: slot r lives in lane r
    if (lane == 0) pr[e] = -1.f;
    __syncwarp();
  }
  total = sum_in_reference_order(chosen, k);  // bit-identical to the reference's sum over the k values
  if (lane < k) {
    ids[m * k + lane] = chosen_id;
    wts[m * k + lane] = norm_topk ? chosen / total : chosen;
  }
}

// Router on the tensor cores without giving up f32 routing: the normalised row v is written
// three times in bf16 -- hi = bf16(v), lo = bf16(v - hi), lo2 = bf16(v - hi - lo), which sum to
// v to within an ulp of f32 -- and multiplied with the (bf16) router matrix repeated three
// times along k.  Every product is exact in f32, only the accumulation order differs from
// the reference's.  One block per token; also writes the plain bf16 row the experts read.
// REDUCE: the rows first receive the addends the ranks pushed for the latest reduction (the
// attention output projection under tensor parallelism), as k_rmsnorm_reduce does.
template <int REDUCE>
__global__ void k_moe_norm_split(float* x, const float* gamma, float eps, int plus_one, int H, __nv_bfloat16* xn,
                                 __nv_bfloat16* xs3, PeerPush px, int32_t* err) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float red[32];
  const int64_t m = blockIdx.x;
  float* row = x + m * H;
  float ss = 0.f;
  if (REDUCE) {
    const uint32_t e = *(volatile uint32_t*)px.epoch;
    const uint32_t par = e & 1u;
    if ((int)threadIdx.x < px.world) peer_wait_flag(px.flags[px.rank] + par * px.world + threadIdx.x, e, err);
    __syncthreads();
    const float* slots = px.data[px.rank] + (int64_t)par * px.world * px.max_elems + m * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float acc = row[i];
      for (int r = 0; r < px.world; ++r) acc += __ldcg(slots + (int64_t)r * px.max_elems + i);
      row[i] = acc;  // read back below by this same thread
      ss += acc * acc;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss += row[i] * row[i];
  }
  ss = block_sum_f(ss, red);
  const float rms = sqrtf(ss / (float)H + eps);
  __nv_bfloat16* o3 = xs3 + m * 3 * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = gamma ? row[i] / rms * (plus_one ? 1.f + gamma[i] : gamma[i]) : row[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo2 = __float2bfloat16_rn(r1 - __bfloat162float(lo));
    xn[m * H + i] = hi;
    o3[i] = hi;
    o3[H + i] = lo;
    o3[2 * H + i] = lo2;
  }
}

// One warp per token: softmax over the router logits, top-k (ties -> lower expert id),
// optional renormalisation.  Dynamic shared memory: E floats per warp.
__global__ void k_moe_topk(const float* logits, int64_t M, int E, int k, int norm_topk, uint32_t* ids, float* wts) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int64_t m = (int64_t)blockIdx.x * nw + wid;
  if (m >= M) return;
  float* pr = sm + (size_t)wid * E;
  const float* lg = logits + m * E;
  float mx = -3.4028234663852886e38f;
  for (int e = lane; e < E; e += 32) {
    const float v = lg[e];
    pr[e] = v;
    mx = fmaxf(mx, v);
  }
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(pr[e] - mx);
    pr[e] = v;
    sum += v;
  }
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) pr[e] = pr[e] / sum;
  __syncwarp();
  float chosen = 0.f, total = 0.f;
  uint32_t chosen_id = 0;
  for (int r = 0; r < k; ++r) {
    unsigned long long best = 0;
    for (int e = lane; e < E; e += 32) {
      const float v = pr[e];
      if (v < 0.f) continue;
      const unsigned long long q = ((unsigned long long)__float_as_uint(v) << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)e);
      best = q > best ? q : best;
    }
    for (int o = 16; o; o >>= 1) {
      const unsigned long long w = __shfl_xor_sync(0xffffffffu, best, o);
      best = w > best ? w : best;
    }
    const uint32_t e = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull);
    const float v = __uint_as_float((uint32_t)(best >> 32));
    if (lane == r) { chosen = v; chosen_id = e; }
    if (lane == 0) pr[e] = -1.f;
    __syncwarp();
  }
  total = sum_in_reference_order(chosen, k);  // bit-identical to the reference's sum over the k values
  if (lane < k) {
    ids[m * k + lane] = chosen_id;
    wts[m * k + lane] = norm_topk ? chosen / total : chosen;
  }
}

// One block of at least El threads (El <= 1024).  Counts the pairs routed to experts
// [e_lo, e_lo + El), lays the groups out back to back, lists the GEMM tiles (tn rows each,
// never crossing a group) and gives every pair its row (or -1 when another rank owns its
// expert).  Thread e owns expert e: two block-wide prefix sums give its first row and its
// first tile.
__global__ void k_moe_plan(const uint32_t* ids, int P, int e_lo, int El, int tn, int32_t* pos, int32_t* tile_expert,
                           int32_t* tile_row0, int32_t* tile_rows, int32_t* n_tiles) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ int sh_i[];
  int* cnt = sh_i;          // [El]
  int* cur = sh_i + El;     // [El]
  __shared__ int wsum_rows[32], wsum_tiles[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  for (int e = tid; e < El; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += blockDim.x) {
    const int e = (int)ids[p] - e_lo;
    if (e >= 0 && e < El) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  const int n = tid < El ? cnt[tid] : 0;
  const int nt = (n + tn - 1) / tn;
  int rows_incl = n, tiles_incl = nt;
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, rows_incl, o), b = __shfl_up_sync(0xffffffffu, tiles_incl, o);
    if (lane >= o) { rows_incl += a; tiles_incl += b; }
  }
  if (lane == 31) { wsum_rows[wid] = rows_incl; wsum_tiles[wid] = tiles_incl; }
  __syncthreads();
  if (wid == 0) {
    int a = wsum_rows[lane], b = wsum_tiles[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int a2 = __shfl_up_sync(0xffffffffu, a, o), b2 = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) { a += a2; b += b2; }
    }
    wsum_rows[lane] = a;
    wsum_tiles[lane] = b;
  }
  __syncthreads();
  const int row0 = rows_incl - n + (wid ? wsum_rows[wid - 1] : 0);
  const int tile0 = tiles_incl - nt + (wid ? wsum_tiles[wid - 1] : 0);
  if (tid < El) {
    cur[tid] = row0;
    for (int t = 0; t < nt; ++t) {
      tile_expert[tile0 + t] = tid;
      tile_row0[tile0 + t] = row0 + t * tn;
      tile_rows[tile0 + t] = min(tn, n - t * tn);
    }
  }
  if (tid == blockDim.x - 1) *n_tiles = tile0 + nt;
  __syncthreads();
  for (int p = tid; p < P; p += blockDim.x) {
    const int e = (int)ids[p] - e_lo;
    pos[p] = (e >= 0 && e < El) ? atomicAdd(&cur[e], 1) : -1;
  }
}

// xg[pos[p], :] = xn[p / k, :] (bf16 rows of H elements, H % 8 == 0)
__global__ void k_moe_gather(const __nv_bfloat16* xn, const int32_t* pos, int64_t P, int k, int H, __nv_bfloat16* xg) {
  // The launch trigger comes AFTER this kernel's own dependency wait: a dependent that starts
  // early can then rely on the planning kernel (this kernel's predecessor) being complete, i.e.
  // read the tile list and stream its expert weights while the rows are still being gathered.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int per = H / 8;
  const int64_t total = P * per;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / per;
    const int j = (int)(i - p * per);
    const int r = pos[p];
    if (r < 0) continue;
    ((uint4*)(xg + (int64_t)r * H))[j] = ((const uint4*)(xn + (p / k) * H))[j];
  }
}

// out[t, :] = (add_residual ? x[t, :] : 0) + sum over slots s of wts[t, s] * y[pos[t k + s], :]
// (out may be x itself)
// PUSH: instead of writing `out`, every rank's exchange area receives this rank's expert sum as
// its addend of the next reduction (no residual: the consumer adds the addends to x).
template <int PUSH>
__global__ void k_moe_combine(const float* y, const int32_t* pos, const float* wts, int64_t M, int k, int H, int add_residual,
                              const float* x, float* out, PeerPush px) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t slot0 = PUSH ? ((int64_t)peer_push_parity(px) * px.world + px.rank) * px.max_elems : 0;
  const int per = H / 4;
  const int64_t total = M * per;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / per;
    const int j = (int)(i - t * per);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < k; ++s) {
      const int r = pos[t * k + s];
      if (r < 0) continue;
      const float w = wts[t * k + s];
      const float4 v = ((const float4*)(y + (int64_t)r * H))[j];
      acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
    }
    if (PUSH) {
      for (int r = 0; r < px.world; ++r) ((float4*)(px.data[r] + slot0 + t * H))[j] = acc;
      continue;
    }
    if (add_residual) {
      const float4 b = ((const float4*)(x + t * H))[j];
      acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    ((float4*)(out + t * H))[j] = acc;
  }
  if (PUSH) {
    __syncthreads();
    if (threadIdx.x == 0) peer_push_done(px, gridDim.x);
  }
}

struct MoeGemmArgs {
  const int32_t* tile_expert;
  const int32_t* tile_row0;
  const int32_t* tile_rows;
  const int32_t* n_tiles;
  void* out;       // DUAL: bf16 [rows, N]; else f32 [rows, N]
  int64_t ldo;
  int N;           // output features per expert
  int w_rows;      // rows one expert occupies in the stacked weight matrix
  int kb_total;
  int act;
  int32_t* err;
};

// One CTA per (128 output features, tile of the list).  Same warp roles and ring as the dense
// tensor-core GEMM: warp 0 lane 0 loads with TMA, warp 1 lane 0 issues the MMAs, warps 2-5
// read the accumulators back.  DUAL keeps two accumulators (gate in TMEM columns [0, TN), up
// in [TN, 2 TN)) fed by the same activation tile.
template <int TN, int DUAL, int STAGES, int MINB>
__global__ void __launch_bounds__(192, MINB)
k_moe_gemm(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_u,
           const __grid_constant__ CUtensorMap map_x, MoeGemmArgs p) {
  constexpr uint32_t W_BYTES = A_BYTES * (DUAL ? 2 : 1);
  constexpr uint32_t B_BYTES = TN * BK * 2;
  constexpr uint32_t STAGE_BYTES = W_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * TN;
  constexpr uint32_t NCOLS = ACC_COLS < 32 ? 32 : ACC_COLS;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The tile list was complete before this kernel could start (k_moe_gather raises its launch
  // trigger only after its wait on the planning kernel), so it is read -- and the weight tiles
  // it names are requested -- before this kernel's own dependency wait; only the gathered
  // activations and the stores wait for the predecessor.
  const int t = blockIdx.y;
  if (t >= *p.n_tiles) return;  // uniform over the CTA, before anything is allocated
  const int expert = p.tile_expert[t], row0 = p.tile_row0[t], rows = p.tile_rows[t];

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  const uint32_t bar_accum = bars + 16 * STAGES;
  uint8_t* gen = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 8);
  volatile int* cta_abort = (volatile int*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 12);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BM;
  const int wrow = expert * p.w_rows + n0;
  const int nkb = p.kb_total;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bars + 8 * s, 2);             // full[s]: weight arrival + activation arrival
      mbar_init(bars + 8 * (STAGES + s), 1);  // empty[s]: one tcgen05.commit
    }
    mbar_init(bar_accum, 1);
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"(NCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  bool acc_ok = false;
  if (warp == 0) {
    if (lane == 0) {
      const int pre = min(nkb, STAGES);
      for (int i = 0; i < pre; ++i) {  // weights of the first stages: no dependency
        const uint32_t full = bars + 8 * i;
        const uint32_t a = base + i * STAGE_BYTES;
        mbar_expect_tx(full, W_BYTES);
        tma_load_2d(a, &map_w, i * BK, wrow, full);
        if (DUAL) tma_load_2d(a + A_BYTES, &map_u, i * BK, wrow, full);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t full = bars + 8 * s;
        const uint32_t a = base + s * STAGE_BYTES;
        const int k = i * BK;
        if (i >= pre) {
          const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
          if (!mbar_wait(bars + 8 * (STAGES + s), ph ^ 1u, cta_abort, p.err)) break;
          mbar_expect_tx(full, W_BYTES);
          tma_load_2d(a, &map_w, k, wrow, full);
          if (DUAL) tma_load_2d(a + A_BYTES, &map_u, k, wrow, full);
        }
        mbar_expect_tx(full, B_BYTES);
        tma_load_2d(a + W_BYTES, &map_x, k, row0, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(TN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(bars + 8 * s, ph, cta_abort, p.err);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = base + s * STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          const uint64_t db = umma_desc(a + W_BYTES + kk * UMMA_K * 2);
          umma_bf16(tmem_acc, umma_desc(a + kk * UMMA_K * 2), db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          if (DUAL) umma_bf16(tmem_acc + TN, umma_desc(a + A_BYTES + kk * UMMA_K * 2), db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bars + 8 * (STAGES + s));
      }
      if (ok) umma_commit(bar_accum);
    }
  } else {
    // the stores belong to the stream order
    asm volatile("griddepcontrol.wait;" ::: "memory");
    acc_ok = mbar_wait(bar_accum, 0, cta_abort, p.err);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  if (warp >= 2 && acc_ok) {
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < TN; c0 += 16) {
      if (c0 >= rows) break;
      uint32_t g[16];
      tmem_ld16(lane_addr + (uint32_t)c0, g);
      if (DUAL) {
        uint32_t u[16];
        tmem_ld16(lane_addr + (uint32_t)(TN + c0), u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j >= rows) break;
            const float a = __uint_as_float(g[j]);
            const float h = (p.act == 0 ? silu_f(a) : gelu_f(a)) * __uint_as_float(u[j]);
            ((__nv_bfloat16*)p.out)[(int64_t)(row0 + c0 + j) * p.ldo + n] = __float2bfloat16_rn(h);
          }
        }
      } else {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j >= rows) break;
            ((float*)p.out)[(int64_t)(row0 + c0 + j) * p.ldo + n] = __uint_as_float(g[j]);
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(NCOLS) : "memory");
  }
}

template <int TN, int DUAL, int STAGES, int MINB>
int launch_moe_gemm(cg_ctx* c, const CUtensorMap& mw, const CUtensorMap& mu, const CUtensorMap& mx, const MoeGemmArgs& a,
                    dim3 grid) {
  constexpr size_t smem = (size_t)STAGES * (A_BYTES * (DUAL ? 2 : 1) + TN * BK * 2) + 1024 + 16 * STAGES + 64;
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_moe_gemm<TN, DUAL, STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  CG_CUDA(c, launch_kernel(c, k_moe_gemm<TN, DUAL, STAGES, MINB>, grid, dim3(192), smem, 1, mw, mu, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

static int launch_combine(cg_ctx* c, const MoeArgs& a) {
  const dim3 grid(grid_for(a.M * (a.H / 4), 256));
  if (a.push) {
    if (a.M * a.H > a.push->max_elems) return fail(c, CG_ERR_INVALID, "moe: rows do not fit the exchange area");
    CG_CUDA(c, launch_kernel(c, k_moe_combine<1>, grid, dim3(256), 0, 1, (const float*)a.w.y, (const int32_t*)a.w.pos,
                             (const float*)a.w.wts, a.M, a.k, a.H, 0, a.x, a.out, *a.push));
  } else {
    CG_CUDA(c, launch_kernel(c, k_moe_combine<0>, grid, dim3(256), 0, 1, (const float*)a.w.y, (const int32_t*)a.w.pos,
                             (const float*)a.w.wts, a.M, a.k, a.H, a.add_residual, a.x, a.out, PeerPush{}));
  }
  CG_LAUNCHED(c);
  return CG_OK;
}

int moe_pick_tn(int64_t pairs, int experts) {
  const int64_t avg = (pairs + experts - 1) / std::max(1, experts);
  return avg <= 8 ? 16 : avg <= 20 ? 32 : avg <= 40 ? 64 : 128;
}

int64_t moe_max_tiles(int64_t pairs, int experts_local, int tn) {
  return std::max<int64_t>(1, std::min<int64_t>(pairs, pairs / tn + experts_local));
}

int moe_ffn(cg_ctx* c, const MoeArgs& a) {
  if (a.M == 0) return CG_OK;
  if (a.k < 1 || a.k > 32 || a.k > a.E) return fail(c, CG_ERR_UNSUPPORTED, "moe: experts per token must be in [1, 32]");
  if (a.push && !a.router3) return fail(c, CG_ERR_INVALID, "moe: the pushed reduction needs the bf16 router path");
  if (a.E > 1024 || a.H % 8 || a.Fe % 8) return fail(c, CG_ERR_UNSUPPORTED, "moe: sizes must be multiples of 8, at most 1024 experts");
  const int64_t P = a.M * a.k;
  if (P > 2147483647ll / 4) return fail(c, CG_ERR_UNSUPPORTED, "moe: too many (token, expert) pairs");
  const int tn = moe_pick_tn(P, a.E);
  const int64_t max_tiles = moe_max_tiles(P, a.El, tn);
  if (max_tiles > 65535) return fail(c, CG_ERR_UNSUPPORTED, "moe: too many tiles");

  if (a.router3) {
    if (a.push)
      CG_CUDA(c, launch_kernel(c, k_moe_norm_split<1>, dim3((unsigned)a.M), dim3(256), 0, 1, a.out, a.gamma, a.eps, a.plus_one, a.H,
                               a.xn, a.xs3, *a.push, c->core->dev_err));
    else
      CG_CUDA(c, launch_kernel(c, k_moe_norm_split<0>, dim3((unsigned)a.M), dim3(256), 0, 1, const_cast<float*>(a.x), a.gamma, a.eps,
                               a.plus_one, a.H, a.xn, a.xs3, PeerPush{}, c->core->dev_err));
    CG_LAUNCHED(c);
    const int64_t K3 = 3 * (int64_t)a.H;
    if (gemm_dec_supported(a.M, K3)) {
      DecGemm g;
      g.x = a.xs3; g.ldx = K3; g.w = a.router3; g.ldw = K3; g.w_rows = a.E;
      g.out = a.logits; g.ldo = a.E; g.residual = nullptr; g.out_mode = 0; g.push = nullptr; g.dual = 0; g.act = 0;
      g.M = a.M; g.N = a.E; g.K = K3;
      CG_TRY(gemm_dec(c, g));
    } else {
      CG_TRY(gemm_tc(c, a.xs3, K3, a.router3, K3, a.logits, a.E, nullptr, a.M, a.E, K3, 0, 0, nullptr));
    }
    const int warps = 4;
    CG_CUDA(c, launch_kernel(c, k_moe_topk, dim3((unsigned)((a.M + warps - 1) / warps)), dim3(32 * warps),
                             (size_t)warps * a.E * 4, 1, (const float*)a.logits, a.M, a.E, a.k, a.norm_topk, a.w.ids, a.w.wts));
    CG_LAUNCHED(c);
  } else {
    const size_t smem = (size_t)(a.H + a.E) * 4;
    static PerDeviceSize configured_on;
  size_t& configured = configured_on.at(c->core->device);
    if (smem > 48 * 1024 && smem > configured) {
      CG_CUDA(c, cudaFuncSetAttribute(k_moe_route, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured = smem;
    }
    CG_CUDA(c, launch_kernel(c, k_moe_route, dim3((unsigned)a.M), dim3(256), smem, 1, a.x, a.gamma, a.eps, a.plus_one, a.router,
                             a.H, a.E, a.k, a.norm_topk, a.xn, a.w.ids, a.w.wts));
    CG_LAUNCHED(c);
  }
  // one thread per local expert is the minimum; more threads only help the histogram of a long prompt
  const unsigned plan_threads = P > 4096 ? 1024u : (unsigned)std::max(128, (a.El + 31) / 32 * 32);
  CG_CUDA(c, launch_kernel(c, k_moe_plan, dim3(1), dim3(plan_threads), (size_t)a.El * 8, 1, (const uint32_t*)a.w.ids, (int)P, a.e_lo,
                           a.El, tn, a.w.pos, a.w.tile_expert, a.w.tile_row0, a.w.tile_rows, a.w.n_tiles));
  CG_LAUNCHED(c);
  CG_CUDA(c, launch_kernel(c, k_moe_gather, dim3(grid_for(P * (a.H / 8), 256)), dim3(256), 0, 1, (const __nv_bfloat16*)a.xn,
                           (const int32_t*)a.w.pos, P, a.k, a.H, a.w.xg));
  CG_LAUNCHED(c);

  MoeGemmArgs g;
  g.tile_expert = a.w.tile_expert;
  g.tile_row0 = a.w.tile_row0;
  g.tile_rows = a.w.tile_rows;
  g.n_tiles = a.w.n_tiles;
  g.act = a.act;
  g.err = c->core->dev_err;
  CUtensorMap mw, mu, mx;
  // gate / up: h[P, Fe] = act(xg Wg^T) * (xg Wu^T)
  CG_TRY(make_map(c, &mw, a.w_gate, (int64_t)a.El * a.Fe, a.H, a.H, BM));
  CG_TRY(make_map(c, &mu, a.w_up, (int64_t)a.El * a.Fe, a.H, a.H, BM));
  CG_TRY(make_map(c, &mx, a.w.xg, P, a.H, a.H, tn));
  g.out = a.w.h; g.ldo = a.Fe; g.N = a.Fe; g.w_rows = a.Fe; g.kb_total = (a.H + BK - 1) / BK;
  dim3 grid((unsigned)((a.Fe + BM - 1) / BM), (unsigned)max_tiles);
  if (tn == 128 && c->opt_persistent) {
    // many rows per expert: the persistent kernel (epilogue overlapped with the next tile)
    CG_TRY(gemm_tcp_grouped(c, a.w.xg, P, a.w_gate, a.w_up, a.El, a.w.h, a.Fe, a.H, 1, a.act, a.w.tile_expert, a.w.tile_row0,
                            a.w.tile_rows, a.w.n_tiles, max_tiles));
    CG_TRY(gemm_tcp_grouped(c, a.w.h, P, a.w_down, nullptr, a.El, a.w.y, a.H, a.Fe, 0, 0, a.w.tile_expert, a.w.tile_row0,
                            a.w.tile_rows, a.w.n_tiles, max_tiles));
    return launch_combine(c, a);
  }
  switch (tn) {
    case 16: CG_TRY((launch_moe_gemm<16, 1, 3, 2>(c, mw, mu, mx, g, grid))); break;
    case 32: CG_TRY((launch_moe_gemm<32, 1, 3, 1>(c, mw, mu, mx, g, grid))); break;
    case 64: CG_TRY((launch_moe_gemm<64, 1, 4, 1>(c, mw, mu, mx, g, grid))); break;
    default: CG_TRY((launch_moe_gemm<128, 1, 4, 1>(c, mw, mu, mx, g, grid))); break;
  }
  // down: y[P, H] = h Wd^T
  CG_TRY(make_map(c, &mw, a.w_down, (int64_t)a.El * a.H, a.Fe, a.Fe, BM));
  CG_TRY(make_map(c, &mx, a.w.h, P, a.Fe, a.Fe, tn));
  g.out = a.w.y; g.ldo = a.H; g.N = a.H; g.w_rows = a.H; g.kb_total = (a.Fe + BK - 1) / BK;
  grid = dim3((unsigned)((a.H + BM - 1) / BM), (unsigned)max_tiles);
  switch (tn) {
    case 16: CG_TRY((launch_moe_gemm<16, 0, 5, 2>(c, mw, mw, mx, g, grid))); break;
    case 32: CG_TRY((launch_moe_gemm<32, 0, 5, 2>(c, mw, mw, mx, g, grid))); break;
    case 64: CG_TRY((launch_moe_gemm<64, 0, 4, 2>(c, mw, mw, mx, g, grid))); break;
    default: CG_TRY((launch_moe_gemm<128, 0, 6, 1>(c, mw, mw, mx, g, grid))); break;
  }
  return launch_combine(c, a);
}

}  // namespace cg

using namespace cg;

extern "C" int32_t cg_fused_moe(cg_ctx* c, const cg_tensor* x, const cg_tensor* router, const cg_tensor* gate,
                                const cg_tensor* up, const cg_tensor* down, int32_t top_k, int32_t norm_topk, int32_t act,
                                cg_tensor** out, cg_tensor** ids_out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !router || !gate || !up || !down || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32 || router->tag != CG_F32 || gate->tag != CG_F32 || up->tag != CG_F32 || down->tag != CG_F32)
    return fail(c, CG_ERR_DTYPE, "moe wants F32 tensors");
  if (x->rank < 1 || router->rank != 2 || gate->rank != 3 || up->rank != 3 || down->rank != 3)
    return fail(c, CG_ERR_SHAPE, "moe: x [.., H], router [E, H], gate/up [E, F, H], down [E, H, F]");
  const int64_t H = x->dims[x->rank - 1], E = router->dims[0], Fe = gate->dims[1];
  const int64_t M = H ? x->numel() / H : 0;
  if (router->dims[1] != H || gate->dims[0] != E || gate->dims[2] != H || up->dims[0] != E || up->dims[1] != Fe ||
      up->dims[2] != H || down->dims[0] != E || down->dims[1] != H || down->dims[2] != Fe)
    return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  if (act != 0 && act != 1) return fail(c, CG_ERR_INVALID, "unknown activation");
  if (top_k < 1 || top_k > E) return fail(c, CG_ERR_SHAPE, "moe: top_k out of range");
  Hold xc, rc, gb, ub, db, r, ids, wts, pos, tiles, xn, xg, h, y, r3, xs3, lgt;
  CG_TRY(as_contiguous_f32(c, x, &xc.t));
  CG_TRY(as_contiguous_f32(c, router, &rc.t));
  for (auto pr : {std::make_pair(gate, &gb), std::make_pair(up, &ub), std::make_pair(down, &db)}) {
    if (pr.first->storage == ST_BF16 && pr.first->contiguous()) { const_cast<cg_tensor*>(pr.first)->rc++; pr.second->t = const_cast<cg_tensor*>(pr.first); }
    else CG_TRY(cg_to_bf16(c, pr.first, &pr.second->t));
  }
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
  const int64_t P = M * top_k;
  int64_t n = std::max<int64_t>(P, 1);
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &ids.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &wts.t));
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &pos.t));
  int64_t nt = 3 * n + 4;
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &nt, 1, &tiles.t));
  int64_t s2[2] = {std::max<int64_t>(M, 1), H};
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &xn.t));
  s2[0] = n;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &xg.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &y.t));
  s2[1] = Fe;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &h.t));
  if (M > 0) {
    CG_CUDA(c, cudaMemsetAsync(xg.t->data(), 0, (size_t)n * H * 2, c->core->stream));
    CG_CUDA(c, cudaMemsetAsync(h.t->data(), 0, (size_t)n * Fe * 2, c->core->stream));
    MoeArgs a;
    a.x = (const float*)xc.t->data();
    a.out = (float*)r.t->data();
    a.gamma = nullptr; a.eps = 0.f; a.plus_one = 0;
    a.router = (const float*)rc.t->data();
    a.router3 = nullptr; a.xs3 = nullptr; a.logits = nullptr;
    if (router->storage == ST_BF16) {
      // bf16 router weights: the split-precision tensor-core router
      Hold rb;
      CG_TRY(cg_to_bf16(c, router, &rb.t));
      int64_t d3[2] = {E, 3 * H};
      CG_TRY(new_tensor(c, CG_F32, ST_BF16, d3, 2, &r3.t));
      for (int rep3 = 0; rep3 < 3; ++rep3)
        CG_CUDA(c, cudaMemcpy2DAsync((__nv_bfloat16*)r3.t->data() + rep3 * H, (size_t)3 * H * 2, rb.t->data(), (size_t)H * 2,
                                     (size_t)H * 2, (size_t)E, cudaMemcpyDeviceToDevice, c->core->stream));
      d3[0] = M;
      CG_TRY(new_tensor(c, CG_F32, ST_BF16, d3, 2, &xs3.t));
      d3[1] = E;
      CG_TRY(new_tensor(c, CG_F32, ST_F32, d3, 2, &lgt.t));
      a.router3 = (const __nv_bfloat16*)r3.t->data();
      a.xs3 = (__nv_bfloat16*)xs3.t->data();
      a.logits = (float*)lgt.t->data();
    }
    a.w_gate = (const __nv_bfloat16*)gb.t->data();
    a.w_up = (const __nv_bfloat16*)ub.t->data();
    a.w_down = (const __nv_bfloat16*)db.t->data();
    a.H = (int)H; a.E = (int)E; a.k = top_k; a.Fe = (int)Fe; a.norm_topk = norm_topk; a.act = act;
    a.e_lo = 0; a.El = (int)E; a.add_residual = 0; a.M = M;
    a.xn = (__nv_bfloat16*)xn.t->data();
    int32_t* t = (int32_t*)tiles.t->data();
    a.w.ids = (uint32_t*)ids.t->data();
    a.w.wts = (float*)wts.t->data();
    a.w.pos = (int32_t*)pos.t->data();
    a.w.tile_expert = t; a.w.tile_row0 = t + n; a.w.tile_rows = t + 2 * n; a.w.n_tiles = t + 3 * n;
    a.w.xg = (__nv_bfloat16*)xg.t->data();
    a.w.h = (__nv_bfloat16*)h.t->data();
    a.w.y = (float*)y.t->data();
    CG_TRY(moe_ffn(c, a));
  }
  if (ids_out) {
    int64_t d2[2] = {M, top_k};
    Hold io;
    CG_TRY(new_tensor(c, CG_U32, ST_U32, d2, 2, &io.t));
    if (P) CG_CUDA(c, cudaMemcpyAsync(io.t->data(), ids.t->data(), (size_t)P * 4, cudaMemcpyDeviceToDevice, c->core->stream));
    *ids_out = io.take();
  }
  *out = r.take();
  return CG_OK;
}
