// gemm_dec.cu — the decode-step GEMM: y[M, N] = x[M, K] w[N, K]^T for M <= 32 tokens.
//
// With a handful of tokens the linear layers of catgrad-llm/src/models/llama.rs:12-115 are
// pure weight streaming, so this kernel is built around keeping HBM busy:
//
//   * warp 0 streams 128-row weight tiles by TMA into a shared-memory ring and starts doing
//     so BEFORE the preceding kernel has finished (programmatic dependent launch): weights
//     do not depend on it.  Only the small bf16 activation tiles wait for the predecessor.
//   * a CTA keeps its shared-memory ring small (about a third of an SM) so that the CTAs of
//     the NEXT GEMM in the stream can already be resident and prefetching their weights while
//     this one computes: the HBM stream does not stop at kernel boundaries.
//   * warp 1 issues tcgen05.mma (128 x TN x 16, f32 accumulators in TMEM).  For the gate/up
//     pair of the FFN both 128-row tiles share the CTA and the epilogue writes
//     act(gate) * up directly (llama.rs:27), so the [M, 2F] intermediate never exists.
//   * split-K partials are PUSHED over distributed shared memory inside a thread-block cluster:
//     every CTA stores its partial rows into the exchange area of the CTA that finishes them,
//     one cluster barrier makes the stores visible, and the owner adds the partials in rank
//     order (deterministic) out of its own shared memory and applies the epilogue (residual add /
//     bf16 / act) once.  No CTA reads another's memory, so none has to wait for the others
//     before it leaves; the residual of the element a thread will finish is fetched while the
//     MMAs still run.
//
//   * two optional hand-overs ride on the epilogue.  Norm hand-over: a residual GEMM also
//     leaves bf16(out * gain) and per-CTA sums of out^2, and the GEMM behind the norm applies
//     1 / rms per row to its accumulators (RMSNorm(x) W^T = (x gain) W^T / rms(x)), so decode
//     steps of pre-norm models run no norm kernels.  Push: under tensor parallelism the partial
//     product goes straight into every rank's mapped exchange area and the last CTA raises
//     this rank's flag there (peer.cuh), instead of a collective call.
//
// All waits are bounded; on expiry the context's error word is raised and the kernel still
// passes its cluster barriers, frees its TMEM and returns.
#include <algorithm>

#include "act.cuh"
#include "kernels.h"
#include "peer.cuh"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

struct DecArgs {
  void* out;
  int64_t ldo;
  const float* residual;
  int out_mode;
  int dual, act, up_off;
  int M, N, K;
  int kb_total, kb_per_split, splits, stages;
  int x_rows;       // activation rows per k block in the ring (8 or TN)
  int xstage_cols;  // split-K: token columns of the exchange area (>= min(TN, M)); 0 without split-K
  int xstage_in_ring;  // the exchange area lies over the ring (more than 16 tokens: it would cost the ring a
                       // stage): then a first cluster barrier says every CTA's ring is idle before anyone pushes
  int32_t* err;
  int trace;  // slot in the timeline buffer, or -1
  PeerPush push;  // out_mode 3
  int total_ctas;
  // norm hand-over (see DecGemm): producer side ...
  __nv_bfloat16* xb_out;
  const float* g_next;
  int g_plus_one;
  float* ss_out;
  // ... and consumer side
  const float* ss_in;
  int ss_parts;
  float ss_inv_h, ss_eps;
};

constexpr int SQ_FLOATS = 2048;  // per-CTA staging of squared outputs (cluster epilogue)

// Timeline of the decode GEMM launches (diagnostics): per slot {first CTA start, predecessor
// complete, last accumulator ready, last CTA end} in globaltimer nanoseconds.
constexpr int TRACE_SLOTS = 2048;
__device__ unsigned long long g_trace[TRACE_SLOTS * 4];

__device__ __forceinline__ void trace_min(int slot, int f) {
  if (slot >= 0) atomicMin(&g_trace[slot * 4 + f], (unsigned long long)globaltimer());
}
__device__ __forceinline__ void trace_max(int slot, int f) {
  if (slot >= 0) atomicMax(&g_trace[slot * 4 + f], (unsigned long long)globaltimer());
}

// `pre` (optional): the residual and next-norm gain of this element, fetched before the accumulator was ready
struct Prefetched {
  bool have;
  float res, gain;
};
__device__ __forceinline__ float finish(const DecArgs& p, int m, int n, float g, float u, uint32_t parity, const float* sc,
                                        const Prefetched pre = Prefetched{false, 0.f, 0.f}) {
  if (p.ss_in) {  // the activations were handed over un-normalised: the row's 1 / rms goes here
    g *= sc[m];
    u *= sc[m];
  }
  float v = g;
  if (p.dual) v = (p.act == 0 ? silu_f(g) : gelu_f(g)) * u;
  const int64_t o = (int64_t)m * p.ldo + n;
  if (p.xb_out) {
    // residual epilogue that also prepares the next norm: the new residual in f32, its
    // gain-scaled bf16 copy for the next GEMM, and its square for the row's sum of squares
    const float r = v + (pre.have ? pre.res : p.residual[o]);
    ((float*)p.out)[o] = r;
    const float gw = pre.have ? pre.gain : p.g_next[n];
    const float gn = p.g_plus_one ? 1.f + gw : gw;
    p.xb_out[o] = __float2bfloat16_rn(r * gn);
    return r * r;
  }
  if (p.out_mode == 3) {
    // this rank's addend goes into slot [parity][rank] of every rank's exchange area
    const int64_t slot = ((int64_t)parity * p.push.world + p.push.rank) * p.push.max_elems + o;
    for (int r = 0; r < p.push.world; ++r) p.push.data[r][slot] = v;
    return 0.f;
  }
  if (p.out_mode == 0) ((float*)p.out)[o] = v;
  else if (p.out_mode == 1) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
  else ((float*)p.out)[o] = v + (pre.have ? pre.res : p.residual[o]);
  return 0.f;
}

// OCC: CTAs per SM the register allocation must allow (the fewer registers a CTA holds, the
// sooner the CTAs of the NEXT kernels in the stream fit beside it and start fetching their weights)
template <int TN, int OCC>
__global__ void __launch_bounds__(192, OCC)
k_gemm_dec(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, DecArgs p) {
  // activation rows fetched per k block: TN, or 8 for up to 8 tokens (the MMA still reads TN rows;
  // the rows past the 8th are whatever follows in shared memory and feed only unused columns)
  const uint32_t X_TILE = (uint32_t)p.x_rows * BK * 2;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const int STAGES = p.stages;
  const uint32_t wbytes = p.dual ? 2 * A_BYTES : A_BYTES;
  const uint32_t stage_bytes = wbytes + X_TILE;
  // split-K exchange area [splits][(1 + dual) * xstage_cols][128 / splits] f32.  Up to 16 tokens it lies
  // behind the ring (not inside it: the other CTAs of the cluster write here while this CTA may
  // still be streaming); above, inside the ring, guarded by one more cluster barrier.
  const uint32_t xbytes = (uint32_t)((p.dual ? 2 : 1) * p.xstage_cols) * BM * 4u;
  const uint32_t xoff = p.xstage_in_ring ? 0u : STAGES * stage_bytes;
  const uint32_t boff = STAGES * stage_bytes + (p.xstage_in_ring ? 0u : xbytes);
  const uint32_t bars = base + boff;  // full[STAGES], empty[STAGES], accum
  const uint32_t bar_accum = bars + 16 * STAGES;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen + boff + 16 * STAGES + 8);
  volatile int* cta_abort = (volatile int*)(gen + boff + 16 * STAGES + 12);
  float* sc = (float*)(gen + boff + 16 * 8 + 64);  // [32] per-token 1 / rms (consumer side)
  // [SQ_FLOATS] squared outputs (producer side): in the ring, which is idle by then (only this
  // CTA touches its ring)
  float* sq = (float*)(gen + (p.xstage_in_ring ? xbytes : 0u));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BM, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_total, kb0 + p.kb_per_split) - kb0;
  const uint32_t ncols = p.dual ? 2 * TN : (TN < 32 ? 32 : TN);
  if (tid == 0) trace_min(p.trace, 0);

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
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  bool acc_ok = false;
  Prefetched pre{false, 0.f, 0.f};
  if (warp == 0) {
    if (lane == 0 && nkb > 0) {
      // weights first: they do not depend on the preceding kernel
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      const int pre = min(nkb, STAGES);
      for (int i = 0; i < pre; ++i) {
        const uint32_t full = bars + 8 * i;
        const uint32_t a = base + i * stage_bytes;
        const int k = (kb0 + i) * BK;
        mbar_expect_tx(full, wbytes);
        tma_load_2d(a, &map_w, k, n0, full);
        if (p.dual) tma_load_2d(a + A_BYTES, &map_w, k, p.up_off + n0, full);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      trace_min(p.trace, 1);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t full = bars + 8 * s;
        const uint32_t a = base + s * stage_bytes;
        const int k = (kb0 + i) * BK;
        if (i >= pre) {
          const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
          if (!mbar_wait(bars + 8 * (STAGES + s), ph ^ 1u, cta_abort, p.err)) break;
          mbar_expect_tx(full, wbytes);
          tma_load_2d(a, &map_w, k, n0, full);
          if (p.dual) tma_load_2d(a + A_BYTES, &map_w, k, p.up_off + n0, full);
        }
        mbar_expect_tx(full, X_TILE);
        tma_load_2d(a + wbytes, &map_x, k, 0, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      const uint32_t idesc = umma_idesc(TN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(bars + 8 * s, ph, cta_abort, p.err);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = base + s * stage_bytes;
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          const uint64_t db = umma_desc(a + wbytes + kk * UMMA_K * 2);
          umma_bf16(tmem_acc, umma_desc(a + kk * UMMA_K * 2), db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          if (p.dual) umma_bf16(tmem_acc + TN, umma_desc(a + A_BYTES + kk * UMMA_K * 2), db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bars + 8 * (STAGES + s));
      }
      if (ok) umma_commit(bar_accum);
    }
  } else {
    // outputs (and the residual) belong to the stream order: wait for the preceding kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (p.splits > 1 && (p.out_mode == 2 || p.xb_out)) {
      // split-K: the element this thread will finish first is known now; fetch its residual (and
      // the next norm's gain) while the MMAs run instead of after the reduction
      const int rows_per = BM / p.splits;
      const int e = tid - 64;
      if (e < rows_per * min(TN, p.M)) {
        const int col = e / rows_per;
        const int n = n0 + split * rows_per + (e - col * rows_per);
        if (n < p.N) {
          asm volatile("ld.global.f32 %0, [%1];" : "=f"(pre.res) : "l"(p.residual + (int64_t)col * p.ldo + n) : "memory");
          if (p.xb_out) asm volatile("ld.global.f32 %0, [%1];" : "=f"(pre.gain) : "l"(p.g_next + n) : "memory");
          pre.have = true;
        }
      }
    }
    if (p.ss_in) {
      // per-token sum of squares = the producer's per-CTA partials added in a fixed order
      // (four interleaved quarters per token, then the quarters): loads fly while the MMAs run
      const int et = tid - 64, m = et >> 2, j = et & 3;
      float a = 0.f;
      if (m < p.M)
        for (int i = j; i < p.ss_parts; i += 4) a += __ldcg(p.ss_in + (int64_t)i * 32 + m);
      const float a1 = __shfl_down_sync(0xffffffffu, a, 1), a2 = __shfl_down_sync(0xffffffffu, a, 2),
                  a3 = __shfl_down_sync(0xffffffffu, a, 3);
      if (j == 0 && m < p.M) sc[m] = 1.0f / sqrtf((((a + a1) + a2) + a3) * p.ss_inv_h + p.ss_eps);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (nkb > 0) {
      acc_ok = mbar_wait(bar_accum, 0, cta_abort, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (tid == 64) trace_max(p.trace, 2);
    }
  }

  const bool cluster = p.splits > 1;
  // the reduction this kernel contributes to: one more than the last one this rank pushed
  // (stable until this kernel's last CTA has seen every other CTA finish)
  uint32_t parity = 0;
  if (p.out_mode == 3 && warp >= 2) parity = peer_push_parity(p.push);
  if (cluster && p.xstage_in_ring) {
    // every thread of every CTA of the cluster is here only after its CTA's loads have landed
    // and its MMAs have read them: from here on the rings may be written by the peers
    __syncwarp();
    cluster_sync_all();
  }
  if (warp >= 2 && acc_ok) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int n = n0 + row;
    // split-K: every value goes straight into the exchange area of the CTA that finishes its row
    // (rows [r * 128 / S, (r + 1) * 128 / S) belong to cluster rank r), slot [this split][col][row]
    const int rows_per = BM / p.splits;
    const int xcols = (p.dual ? 2 : 1) * p.xstage_cols;
    uint32_t xdst = 0;
    if (cluster) {
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(xdst) : "r"(base + xoff), "r"((uint32_t)(row / rows_per)));
      xdst += (uint32_t)(split * xcols * rows_per + row % rows_per) * 4u;
    }
#pragma unroll 1
    for (int c0 = 0; c0 < TN; c0 += 16) {
      if (c0 >= p.M) break;
      uint32_t g[16], u[16];
      tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, g);
      if (p.dual) tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(TN + c0), u);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (cluster) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j >= p.M) break;
          asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(xdst + (uint32_t)((c0 + j) * rows_per) * 4u), "r"(g[j]) : "memory");
          if (p.dual)
            asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(xdst + (uint32_t)((p.xstage_cols + c0 + j) * rows_per) * 4u), "r"(u[j])
                         : "memory");
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j >= p.M) break;
          float r2 = 0.f;
          if (n < p.N) r2 = finish(p, c0 + j, n, __uint_as_float(g[j]), p.dual ? __uint_as_float(u[j]) : 0.f, parity, sc);
          if (p.ss_out) {
            // one CTA per tile here: the tile's 128 rows are summed per token, warp tree then warps in order
            for (int o = 16; o; o >>= 1) r2 += __shfl_xor_sync(0xffffffffu, r2, o);
            if (lane == 0) sq[q * 32 + c0 + j] = r2;
          }
        }
      }
    }
  }
  if (warp >= 2 && p.ss_out && !cluster) {
    // (outside the branch above: all four epilogue warps must reach this barrier)
    asm volatile("bar.sync 2, 128;" ::: "memory");
    const int et = tid - 64;
    if (acc_ok && et < p.M) p.ss_out[(int64_t)blockIdx.x * 32 + et] = ((sq[et] + sq[32 + et]) + sq[64 + et]) + sq[96 + et];
  }

  if (cluster) {
    // One cluster barrier: every CTA's pushes are visible after it, and nobody touches another
    // CTA's shared memory again, so a CTA may leave as soon as its own rows are finished.
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2 && !*cta_abort) {
      const int S = p.splits;
      const int rows_per = BM / S;
      const int cols = min(TN, p.M);
      const int xcols = (p.dual ? 2 : 1) * p.xstage_cols;
      const float* xs = (const float*)(gen + xoff);
      for (int e = tid - 64; e < rows_per * cols; e += 128) {
        const int col = e / rows_per, rl = e - col * rows_per;
        const int row = split * rows_per + rl;
        // the splits' partial sums in rank order (all loads first)
        float pg[16], pu[16];
#pragma unroll
        for (int s = 0; s < 16; ++s) {
          pg[s] = s < S ? xs[(s * xcols + col) * rows_per + rl] : 0.f;
          pu[s] = (p.dual && s < S) ? xs[(s * xcols + p.xstage_cols + col) * rows_per + rl] : 0.f;
        }
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int s = 0; s < 16; ++s) { g += pg[s]; u += pu[s]; }  // the zeros of absent ranks change nothing
        const int n = n0 + row;
        float r2 = 0.f;
        if (n < p.N) r2 = finish(p, col, n, g, u, parity, sc, e == tid - 64 ? pre : Prefetched{false, 0.f, 0.f});
        if (p.ss_out) sq[e] = r2;  // e = col * rows_per + local row
      }
      if (p.ss_out) {
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const int et = tid - 64;
        if (et < cols) {
          float a = 0.f;
          for (int i = 0; i < rows_per; ++i) a += sq[et * rows_per + i];
          p.ss_out[((int64_t)blockIdx.x * S + split) * 32 + et] = a;
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(ncols) : "memory");
  }
  // every thread's pushes precede the barrier above
  if (p.out_mode == 3 && tid == 0) peer_push_done(p.push, (unsigned)p.total_ctas);
  if (tid == 0) trace_max(p.trace, 3);
}

template <int TN, int OCC>
int launch_dec(cg_ctx* c, const CUtensorMap& mw, const CUtensorMap& mx, const DecArgs& a, dim3 grid, size_t smem) {
  static PerDeviceSize configured_on;
  size_t& configured = configured_on.at(c->core->device);
  if (smem > configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_gemm_dec<TN, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CG_CUDA(c, cudaFuncSetAttribute(k_gemm_dec<TN, OCC>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    configured = smem;
  }
  CG_CUDA(c, launch_kernel(c, k_gemm_dec<TN, OCC>, grid, dim3(192), smem, a.splits, mw, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

bool gemm_dec_supported(int64_t M, int64_t K) { return M >= 1 && M <= 32 && K % 8 == 0; }

// split-K: a power of two up to 16 (one cluster; above 8 is the non-portable size this GPU
// supports), at most about three CTAs per SM in total, at least two k blocks per CTA
static int dec_splits(int64_t tiles, int kb_total) {
  // (caps of 300 / 222 / 160 CTAs were measured 0.5 / 9 / 13 % slower per decode step, 600 4 % slower)
  const int cap = 3 * 148;
  int splits = 1;
  while (splits < 16 && tiles * (splits * 2) <= cap && kb_total / (splits * 2) >= 2) splits *= 2;
  const int kb_per = (kb_total + splits - 1) / splits;
  if ((kb_total + kb_per - 1) / kb_per != splits) splits = 1;  // an empty slice would break the cluster shape
  return splits;
}

int gemm_dec_ss_parts(int64_t N, int64_t K) {
  const int64_t tiles = (N + BM - 1) / BM;
  return (int)(tiles * dec_splits(tiles, (int)((K + BK - 1) / BK)));
}

int gemm_dec(cg_ctx* c, const DecGemm& g) {
  if (g.M <= 0 || g.N <= 0) return CG_OK;
  if (!gemm_dec_supported(g.M, g.K) || g.K <= 0 || g.ldw % 8 || g.ldx % 8 || ((uintptr_t)g.w % 16) || ((uintptr_t)g.x % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_dec: unsupported shape or alignment");
  const int tn = g.M <= 16 ? 16 : 32;
  const int64_t tiles = (g.N + BM - 1) / BM;
  const int kb_total = (int)((g.K + BK - 1) / BK);
  const int splits = dec_splits(tiles, kb_total);
  const int kb_per = (kb_total + splits - 1) / splits;
  const size_t wbytes = g.dual ? 2 * A_BYTES : A_BYTES;
  // up to 8 tokens: an 8-row activation box (1 KB instead of 2 per k block), which is what lets a
  // fourth ring stage fit beside the exchange area at three CTAs per SM
  const int x_rows = g.M <= 8 ? 8 : tn;
  const size_t stage = wbytes + (size_t)x_rows * BK * 2;
  // about a third of an SM's shared memory per CTA, so the next GEMM's CTAs can be resident
  // (and prefetching their weights) while this one computes
  // (the paired gate/up GEMM carries two weight tiles per stage, so the same budget would
  // leave it only two stages: it gets three, at two CTAs per SM)
  // The split-K exchange area (written by the other CTAs of the cluster, so outside the ring)
  // comes out of the same budget: three CTAs per SM may use 75 KB each, two 113 KB each.
  const int xstage_cols = splits > 1 ? (int)std::min<int64_t>(tn, g.M) : 0;
  const bool x_in_ring = tn == 32;  // above 16 tokens a separate area would cost the ring a stage (measured: 3 % per step)
  const size_t xarea = (size_t)(g.dual ? 2 : 1) * xstage_cols * BM * 4;
  const size_t xbytes = x_in_ring ? 0 : xarea;
  // (with the 8-row box the MMA of the last stage reads 1 KB past its activation slot: keep that inside the allocation)
  const size_t fixed = 1024 + 16 * 8 + 64 + 128 + (x_rows < tn ? 1024 : 0);
  // (smaller budgets -- 57 or 43 KB, 78 KB for the pair -- were measured 2-5 % slower per step)
  const size_t budget = (g.dual ? 113 * 1024 : 75 * 1024) - fixed;
  int stages = (int)std::max<size_t>(2, (budget > xbytes ? budget - xbytes : 0) / stage);
  // The paired kernel: three stages leave room for two CTAs per SM and nothing else, so when its
  // CTAs fill nearly all of those slots it takes two stages, and the next kernel's CTAs fit beside it
  // and fetch their weights early (Gemma-2-2B shape, 288 CTAs: 2.40 -> 2.25 ms per step; the
  // Llama-3.2-1B shape, 256 CTAs, measured 1-2 % better with three).
  if (g.dual && tiles * splits > 7 * 148 / 4) stages = std::min(stages, 2);
  stages = std::min(stages, std::max(kb_per, 2));
  stages = std::min(stages, 8);
  // the squared-output staging of the norm hand-over lives in the ring
  while ((g.ss_out || x_in_ring) && (x_in_ring ? xarea : 0) + (g.ss_out ? (size_t)SQ_FLOATS * 4 : 0) > (size_t)stages * stage) ++stages;
  const size_t smem = (size_t)stages * stage + xbytes + fixed;

  CUtensorMap mw, mx;
  CG_TRY(make_map(c, &mw, g.w, g.w_rows, g.K, g.ldw, BM));
  CG_TRY(make_map(c, &mx, g.x, g.M, g.K, g.ldx, x_rows));
  DecArgs a;
  a.out = g.out; a.ldo = g.ldo; a.residual = g.residual; a.out_mode = g.out_mode;
  a.dual = g.dual; a.act = g.act; a.up_off = (int)g.N;
  a.M = (int)g.M; a.N = (int)g.N; a.K = (int)g.K;
  a.kb_total = kb_total; a.kb_per_split = kb_per; a.splits = splits; a.stages = stages;
  a.x_rows = x_rows;
  a.xstage_cols = xstage_cols;
  a.xstage_in_ring = x_in_ring && splits > 1 ? 1 : 0;
  a.err = c->core->dev_err;
  a.trace = c->trace_on ? (int)(c->trace_next++ % TRACE_SLOTS) : -1;
  a.total_ctas = (int)(tiles * splits);
  a.xb_out = g.xb_out; a.g_next = g.g_next; a.g_plus_one = g.g_plus_one; a.ss_out = g.ss_out;
  a.ss_in = g.ss_in; a.ss_parts = g.ss_parts; a.ss_inv_h = g.ss_in ? 1.0f / (float)g.K : 0.f; a.ss_eps = g.ss_eps;
  if (g.xb_out && (g.out_mode != 2 || g.dual || !g.g_next || !g.ss_out || g.ldo != g.N))
    return fail(c, CG_ERR_INVALID, "gemm_dec: the norm hand-over needs the residual epilogue on a dense output");
  if (g.out_mode == 3) {
    if (!g.push || g.dual || g.M * g.ldo > g.push->max_elems)
      return fail(c, CG_ERR_INVALID, "gemm_dec: the pushed addend does not fit the exchange area");
    a.push = *g.push;
  } else {
    a.push = PeerPush{};
  }
  dim3 grid((unsigned)tiles, 1, (unsigned)splits);
  // (register bound for 4 CTAs per SM: 0.861 -> 0.836 ms per Llama-3.2-1B decode step against a
  // bound for 3; bounds for 5 and 6 measured the same as 4)
  if (tn == 16) return launch_dec<16, 4>(c, mw, mx, a, grid, smem);
  return launch_dec<32, 4>(c, mw, mx, a, grid, smem);
}

}  // namespace cg

using namespace cg;

extern "C" int32_t cg_trace_enable(cg_ctx* c, int32_t on) {
  if (!c) return CG_ERR_INVALID;
  c->trace_on = on != 0;
  c->trace_next = 0;
  if (on) {
    std::vector<unsigned long long> init((size_t)TRACE_SLOTS * 4);
    for (int i = 0; i < TRACE_SLOTS; ++i) {
      init[i * 4 + 0] = init[i * 4 + 1] = ~0ull;
      init[i * 4 + 2] = init[i * 4 + 3] = 0ull;
    }
    CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
    CG_CUDA(c, cudaMemcpyToSymbol(g_trace, init.data(), init.size() * 8));
  }
  return CG_OK;
}

extern "C" int32_t cg_trace_read(cg_ctx* c, uint64_t* out, int32_t slots) {
  if (!c || !out || slots < 0 || slots > TRACE_SLOTS) return CG_ERR_INVALID;
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  CG_CUDA(c, cudaMemcpyFromSymbol(out, g_trace, (size_t)slots * 32));
  return CG_OK;
}
