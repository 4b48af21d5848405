// gemm_tc.cu — bf16 GEMM on the Blackwell tensor cores: y[M,N] = x[M,K] w[N,K]^T.
//
// The weight is consumed as the checkpoints store it ([out, in], k unit-stride), so the
// `transpose` + `reshape` of catgrad's linear layer (catgrad/src/stdlib/nn/mod.rs:174-199)
// never touches memory.  The operands are swapped on the way into the instruction: a
// 128-row tile of W is the MMA's M side and a tile of TN tokens its N side, so one
// kernel serves decode (TN = 16, HBM-bound weight streaming with split-K) and prefill
// (TN = 256, tensor-bound).
//
// Pipeline per CTA (192 threads):
//   warp 0      one lane issues TMA loads (128B-swizzled [rows, 64] bf16 boxes) into a
//               ring of STAGES shared-memory slots, signalled through mbarriers
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (128 x TN x 16, f32 accumulate
//               in TMEM) and commits slot releases / the final "accumulator ready"
//   warps 2-5   epilogue: tcgen05.ld the accumulator (lane = output feature, column =
//               token) and store coalesced along the feature axis
//
// Weights never depend on the kernel that ran before, so under programmatic dependent
// launch the producer fills the ring with weight tiles BEFORE it waits for the preceding
// kernel; only activation tiles, the residual and the stores come after the wait.  HBM keeps
// streaming while the small kernels between two GEMMs run.
//
// Split-K: the `splits` CTAs that share an output tile form a thread-block cluster; each
// leaves its partial tile in its own shared memory and, after a cluster barrier, CTA r sums
// rows [r * 128 / splits, ...) of all partials over distributed shared memory in rank
// order (deterministic) and stores them.  No partials in HBM, no second kernel.
//
// Every mbarrier wait is bounded (about one second); on expiry the kernel raises the
// context's error word, still passes its cluster barriers, frees its TMEM and returns.
#include <algorithm>

#include "act.cuh"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

struct TcArgs {
  void* out;
  const float* residual;
  float* partial;  // only when splits > 1 without a cluster
  int64_t ldo;
  int M, N, K;
  int out_mode;  // 0 f32, 1 bf16, 2 f32 + residual
  int kb_total, kb_per_split, splits;
  int cluster;   // 1: the splits of a tile are one cluster and reduce over shared memory
  // two accumulators per CTA (ACC2 kernels): the second weight tile starts row2_off rows below
  // the first and both multiply the same activation tile
  int n_stride;  // weight rows between consecutive CTAs along x (128, or 256 for a 256-row tile)
  int row2_off;  // 128: one 256-row tile; N: gate and up rows paired
  int pair_act;  // -1: store both accumulators; 0 / 1: out = act(first) * second in bf16 (silu / tanh-gelu)
  int32_t* err;
};

__device__ __forceinline__ void store_out(const TcArgs& p, int m, int n, float acc) {
  const int64_t o = (int64_t)m * p.ldo + n;
  if (p.out_mode == 0) ((float*)p.out)[o] = acc;
  else if (p.out_mode == 1) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(acc);
  else ((float*)p.out)[o] = acc + p.residual[o];
}

template <int TN, int STAGES, int MINB, int ACC2>
__global__ void __launch_bounds__(192, MINB)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcArgs p) {
  constexpr uint32_t B_BYTES = TN * BK * 2;
  constexpr uint32_t W_BYTES = A_BYTES * (1 + ACC2);
  constexpr uint32_t STAGE_BYTES = W_BYTES + B_BYTES;
  constexpr uint32_t NCOLS = TN * (1 + ACC2) < 32 ? 32 : TN * (1 + ACC2);  // TMEM columns: power of two >= 32

  // the next kernel in the stream may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  const uint32_t bar_accum = bars + 16 * STAGES;
  uint8_t* gen = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 8);
  volatile int* cta_abort = (volatile int*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 12);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * (ACC2 ? p.n_stride : BM), m0 = blockIdx.y * TN, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

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

  bool acc_ok = false;  // epilogue warps: the accumulator is complete
  if (warp == 0) {
    if (lane == 0 && nkb > 0) {
      // weights first: they do not depend on the preceding kernel
      const int pre = min(nkb, STAGES);
      for (int i = 0; i < pre; ++i) {
        const uint32_t full = bars + 8 * i;
        mbar_expect_tx(full, W_BYTES);
        tma_load_2d(base + i * STAGE_BYTES, &map_w, (kb0 + i) * BK, n0, full);
        if (ACC2) tma_load_2d(base + i * STAGE_BYTES + A_BYTES, &map_w, (kb0 + i) * BK, n0 + p.row2_off, full);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t full = bars + 8 * s;
        const uint32_t a = base + s * STAGE_BYTES;
        const int k = (kb0 + i) * BK;
        if (i >= pre) {
          const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
          if (!mbar_wait(bars + 8 * (STAGES + s), ph ^ 1u, cta_abort, p.err)) break;
          mbar_expect_tx(full, W_BYTES);
          tma_load_2d(a, &map_w, k, n0, full);
          if (ACC2) tma_load_2d(a + A_BYTES, &map_w, k, n0 + p.row2_off, full);
        }
        mbar_expect_tx(full, B_BYTES);
        tma_load_2d(a + W_BYTES, &map_x, k, m0, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
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
          const uint64_t da = umma_desc(a + kk * UMMA_K * 2);
          const uint64_t db = umma_desc(a + W_BYTES + kk * UMMA_K * 2);
          umma_bf16(tmem_acc, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          if (ACC2) umma_bf16(tmem_acc + TN, umma_desc(a + A_BYTES + kk * UMMA_K * 2), db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bars + 8 * (STAGES + s));  // slot reusable once these MMAs have read it
      }
      if (ok) umma_commit(bar_accum);
    }
  } else {
    // outputs (and the residual) belong to the stream order: wait for the preceding kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (nkb > 0) {
      acc_ok = mbar_wait(bar_accum, 0, cta_abort, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
  }

  if (warp >= 2 && acc_ok) {
    // TMEM lanes a warp may read: 32 * (warp id mod 4)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int n = n0 + row;
    float* stage = (float*)gen;  // [TN][128] partial tile; the ring is idle by now
#pragma unroll 1
    for (int c0 = 0; c0 < TN; c0 += 16) {
      if (m0 + c0 >= p.M) break;
      uint32_t v[16];
      tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
      if (ACC2) {
        // splits == 1 here: the two accumulators go straight to the output
        uint32_t u[16];
        tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(TN + c0), u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (p.pair_act >= 0) {
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c0 + j;
              if (m >= p.M) break;
              const float g = __uint_as_float(v[j]);
              const float h = (p.pair_act == 0 ? silu_f(g) : gelu_f(g)) * __uint_as_float(u[j]);
              ((__nv_bfloat16*)p.out)[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(h);
            }
          }
        } else {
          const int n2 = n + p.row2_off;
          float res[16], res2[16];
          if (p.out_mode == 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c0 + j;
              res[j] = (m < p.M && n < p.N) ? p.residual[(int64_t)m * p.ldo + n] : 0.f;
              res2[j] = (m < p.M && n2 < p.N) ? p.residual[(int64_t)m * p.ldo + n2] : 0.f;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m >= p.M) break;
            const float a1 = __uint_as_float(v[j]), a2 = __uint_as_float(u[j]);
            const int64_t o = (int64_t)m * p.ldo;
            if (p.out_mode == 1) {
              if (n < p.N) ((__nv_bfloat16*)p.out)[o + n] = __float2bfloat16_rn(a1);
              if (n2 < p.N) ((__nv_bfloat16*)p.out)[o + n2] = __float2bfloat16_rn(a2);
            } else {
              if (n < p.N) ((float*)p.out)[o + n] = p.out_mode == 2 ? a1 + res[j] : a1;
              if (n2 < p.N) ((float*)p.out)[o + n2] = p.out_mode == 2 ? a2 + res2[j] : a2;
            }
          }
        }
        continue;
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (p.cluster) {
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[(c0 + j) * BM + row] = __uint_as_float(v[j]);
      } else if (n < p.N) {
        if (p.splits == 1 && p.out_mode == 2) {
          // out may alias residual, so the compiler cannot move a load above the previous
          // store: issue all 16 residual loads first, then the stores
          float res[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            res[j] = m < p.M ? p.residual[(int64_t)m * p.ldo + n] : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < p.M) ((float*)p.out)[(int64_t)m * p.ldo + n] = __uint_as_float(v[j]) + res[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m >= p.M) break;
            const float acc = __uint_as_float(v[j]);
            if (p.splits > 1) p.partial[((int64_t)split * p.M + m) * p.N + n] = acc;
            else store_out(p, m, n, acc);
          }
        }
      }
    }
  }

  if (p.cluster) {
    // all partial tiles of this output tile are in their CTAs' shared memory
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2 && !*cta_abort) {
      const int S = p.splits;
      const int rows_per = BM / S;
      const int cols = min(TN, p.M - m0);
      const uint32_t stage_u = base;
      for (int e = tid - 64; e < rows_per * cols; e += 128) {
        const int col = e / rows_per;
        const int row = split * rows_per + (e - col * rows_per);
        const float acc = sum_cluster_f32(stage_u + (uint32_t)(col * BM + row) * 4u, S);
        const int n = n0 + row;
        if (n < p.N) store_out(p, m0 + col, n, acc);
      }
    }
    __syncwarp();
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(NCOLS) : "memory");
  }
}

// out = sum over splits of partial (+ residual), in the output precision (only used when the
// splits of a tile could not form a cluster).
__global__ void k_splitk_reduce(const float* partial, int splits, int64_t M, int64_t N, void* out, int64_t ldo,
                                const float* residual, int out_mode) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t total = M * N;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(int64_t)s * total + i];
    const int64_t m = i / N, n = i - m * N;
    const int64_t o = m * ldo + n;
    if (out_mode == 0) ((float*)out)[o] = acc;
    else if (out_mode == 1) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(acc);
    else ((float*)out)[o] = acc + residual[o];
  }
}

template <int TN, int STAGES, int MINB, int ACC2 = 0>
int launch(cg_ctx* c, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, dim3 grid) {
  constexpr size_t smem = (size_t)STAGES * (A_BYTES * (1 + ACC2) + TN * BK * 2) + 1024 + 16 * STAGES + 64;
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_gemm_tc<TN, STAGES, MINB, ACC2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  CG_CUDA(c, launch_kernel(c, k_gemm_tc<TN, STAGES, MINB, ACC2>, grid, dim3(192), smem, a.cluster ? a.splits : 1, mw, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

int pick_tn(int64_t M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

}  // namespace

int gemm_tc_pick_splits(int64_t M, int64_t N, int64_t K) {
  const int tn = pick_tn(M);
  const int64_t tiles = ((N + BM - 1) / BM) * ((M + tn - 1) / tn);
  const int64_t kb = (K + BK - 1) / BK;
  if (tiles >= 148 || kb < 8) return 1;
  // a power of two up to 8 (one portable cluster), at least two k blocks per slice
  int s = 1;
  while (s < 8 && tiles * (s * 2) <= 2 * 148 + 32 && kb / (s * 2) >= 2) s *= 2;
  return s;
}

int gemm_tc_pair(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, __nv_bfloat16* out,
                 int64_t ldo, int64_t M, int64_t F, int64_t K, int act) {
  if (M <= 0 || F <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: k and leading dimensions must be multiples of 8, bases 16-byte aligned");
  if (M > 2147483647ll / 2 || F > 2147483647ll / 4) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: problem too large");
  if (c->opt_persistent && ((c->opt_pair_cta == 2 && gemm_tcp2_supported(F, 1)) || (c->opt_pair_cta && gemm_tcp2_wanted(M, F, K, 1))))
    return gemm_tcp2(c, x, ldx, w, ldw, 2 * F, out, ldo, nullptr, M, F, K, 1, 1, act);
  if (c->opt_persistent && gemm_tcp_wanted(M, F, K)) return gemm_tcp(c, x, ldx, w, ldw, 2 * F, out, ldo, nullptr, M, F, K, 1, 1, act);
  const int tn = M <= 128 ? 128 : 256;
  CUtensorMap mw, mx;
  CG_TRY(make_map(c, &mw, w, 2 * F, K, ldw, BM));
  CG_TRY(make_map(c, &mx, x, M, K, ldx, tn));
  TcArgs a{};
  a.out = out; a.residual = nullptr; a.partial = nullptr; a.ldo = ldo;
  a.M = (int)M; a.N = (int)F; a.K = (int)K; a.out_mode = 1;
  a.kb_total = (int)((K + BK - 1) / BK); a.kb_per_split = a.kb_total; a.splits = 1; a.cluster = 0;
  a.n_stride = BM; a.row2_off = (int)F; a.pair_act = act;
  a.err = c->core->dev_err;
  dim3 grid((unsigned)((F + BM - 1) / BM), (unsigned)((M + tn - 1) / tn), 1);
  if (grid.y > 65535) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: too many token tiles");
  if (tn == 128) CG_TRY((launch<128, 4, 1, 1>(c, mw, mx, a, grid)));
  else CG_TRY((launch<256, 3, 1, 1>(c, mw, mx, a, grid)));
  return CG_OK;
}

int gemm_tc(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, void* out, int64_t ldo,
            const float* residual, int64_t M, int64_t N, int64_t K, int out_mode, int splits, float* workspace) {
  if (M <= 0 || N <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: k and leading dimensions must be multiples of 8, bases 16-byte aligned");
  if (M > 2147483647ll / 2 || N > 2147483647ll / 2) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: problem too large");
  if (c->opt_persistent && splits <= 1 && (c->opt_pair_cta == 2 || (c->opt_pair_cta && gemm_tcp2_wanted(M, N, K, 0))))
    return gemm_tcp2(c, x, ldx, w, ldw, N, out, ldo, residual, M, N, K, out_mode, 0, 0);
  if (c->opt_persistent && splits <= 1 && gemm_tcp_wanted(M, N, K))
    return gemm_tcp(c, x, ldx, w, ldw, N, out, ldo, residual, M, N, K, out_mode, 0, 0);
  const int tn = pick_tn(M);
  const int kb_total = (int)((K + BK - 1) / BK);
  if (splits <= 0) splits = gemm_tc_pick_splits(M, N, K);
  splits = std::min(splits, kb_total);
  int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;  // no empty slices
  // a cluster needs a power-of-two size up to 8 and a tile that fits the staging area
  const bool cluster = splits > 1 && splits <= 8 && (splits & (splits - 1)) == 0 && tn <= 64;

  Hold ws;
  if (splits > 1 && !cluster && !workspace) {
    // A block taken from the caching allocator here is recycled when this call returns; a graph
    // captured now would keep writing to it on every replay, whoever owns it by then.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(c->core->stream, &cap);
    if (cap != cudaStreamCaptureStatusNone)
      return fail(c, CG_ERR_INVALID, "gemm_tc: split-K workspace must be passed in while the stream is being captured");
    int64_t n = (int64_t)splits * M * N;
    CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &ws.t));
    workspace = (float*)ws.t->data();
  }

  CUtensorMap mw, mx;
  CG_TRY(make_map(c, &mw, w, N, K, ldw, BM));
  CG_TRY(make_map(c, &mx, x, M, K, ldx, tn));

  TcArgs a;
  a.out = out;
  a.residual = residual;
  a.partial = workspace;
  a.ldo = ldo;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  a.out_mode = out_mode;
  a.kb_total = kb_total;
  a.kb_per_split = kb_per;
  a.splits = splits;
  a.cluster = cluster ? 1 : 0;
  a.n_stride = BM; a.row2_off = BM; a.pair_act = -1;
  a.err = c->core->dev_err;
  dim3 grid((unsigned)((N + BM - 1) / BM), (unsigned)((M + tn - 1) / tn), (unsigned)splits);
  if (grid.y > 65535) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tc: too many token tiles");
  // large problems: 256 weight rows per CTA in two accumulators, so every activation tile read
  // from L2 feeds twice the math; only while that still leaves a tile for every SM
  if (splits == 1 && tn >= 128 && ((N + 2 * BM - 1) / (2 * BM)) * (int64_t)grid.y >= 148) {
    a.n_stride = 2 * BM;
    grid.x = (unsigned)((N + 2 * BM - 1) / (2 * BM));
    if (tn == 128) CG_TRY((launch<128, 4, 1, 1>(c, mw, mx, a, grid)));
    else CG_TRY((launch<256, 3, 1, 1>(c, mw, mx, a, grid)));
    return CG_OK;
  }
  switch (tn) {
    case 16: CG_TRY((launch<16, 6, 2>(c, mw, mx, a, grid))); break;
    case 32: CG_TRY((launch<32, 5, 2>(c, mw, mx, a, grid))); break;
    case 64: CG_TRY((launch<64, 4, 2>(c, mw, mx, a, grid))); break;
    case 128: CG_TRY((launch<128, 6, 1>(c, mw, mx, a, grid))); break;
    default: CG_TRY((launch<256, 4, 1>(c, mw, mx, a, grid))); break;
  }
  if (splits > 1 && !cluster) {
    CG_CUDA(c, launch_kernel(c, k_splitk_reduce, dim3(grid_for(M * N, 256)), dim3(256), 0, 1, (const float*)workspace, splits,
                             M, N, out, ldo, residual, out_mode));
    CG_LAUNCHED(c);
  }
  return CG_OK;
}

}  // namespace cg
