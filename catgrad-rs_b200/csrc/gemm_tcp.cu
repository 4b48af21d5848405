// gemm_tcp.cu — persistent bf16 GEMM for many tokens (prefill): y[M,N] = x[M,K] w[N,K]^T.
//
// Same operand orientation as gemm_tc.cu (a 128-row tile of W is the MMA's M side, a tile of
// TN tokens its N side), but a CTA stays on its SM and walks a list of output tiles, with the
// accumulator double-buffered in TMEM: while the four epilogue warps read tile i out of one
// half of TMEM and store it, the MMA warp already accumulates tile i+1 into the other half,
// and the TMA warp runs ahead through the shared-memory ring across tile boundaries.  The
// per-tile set-up (TMEM allocation, barrier initialisation, pipeline fill) and the epilogue
// leave the critical path; only the first fill and the last drain of a CTA remain.
//
//   warp 0      TMA producer over all tiles of the CTA (ring of STAGES slots)
//   warp 1      tcgen05.mma issue; commits slot releases and "accumulator full"
//   warps 2-5   epilogue; arrive on "accumulator empty" when a half has been read
//
// PAIR: every tile holds two accumulators fed by the same activation tile -- the gate rows
// and the matching up rows of the FFN -- and the epilogue stores act(gate) * up in bf16
// (catgrad-llm/src/models/llama.rs:27), so the [M, 2F] intermediate never reaches HBM.
//
// Tiles are numbered with the token tile fastest, so the CTAs that run side by side share
// one weight tile (one HBM read, served to the others from L2) while the activations, which
// are far smaller than L2, stay resident.
//
// Every mbarrier wait is bounded; on expiry the kernel raises the context's error word, all
// roles leave their loops, TMEM is freed and the kernel returns.
#include <algorithm>

#include "act.cuh"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

struct TcpArgs {
  void* out;
  const float* residual;
  int64_t ldo;
  int M, N, K;
  int out_mode;   // 0 f32, 1 bf16, 2 f32 + residual (residual may alias out)
  int kb_total;
  int m_tiles, n_tiles;
  int row2_off;   // PAIR: rows between a gate row and its up row
  int act;        // PAIR: 0 silu, 1 tanh-gelu
  // GROUPED (mixture-of-experts): token tiles come from a device-built list, each belonging to
  // one expert whose weights start at row expert * w_rows of the stacked matrix; rows of a tile
  // past `tile_rows` belong to other experts and are not stored
  const int32_t* tile_expert;
  const int32_t* tile_row0;
  const int32_t* tile_rows;
  const int32_t* n_list;
  int w_rows;
  int32_t* err;
};

struct TileAt {
  int m0, m_end, n0, wrow;
};

template <int TN, int GROUPED>
__device__ __forceinline__ TileAt tile_at(const TcpArgs& p, int t) {
  TileAt a;
  if (GROUPED) {
    const int te = t / p.n_tiles;
    a.n0 = (t - te * p.n_tiles) * BM;
    a.m0 = p.tile_row0[te];
    a.m_end = a.m0 + p.tile_rows[te];
    a.wrow = p.tile_expert[te] * p.w_rows + a.n0;
  } else {
    a.m0 = (t % p.m_tiles) * TN;
    a.m_end = p.M;
    a.n0 = (t / p.m_tiles) * BM;
    a.wrow = a.n0;
  }
  return a;
}

template <int TN, int PAIR, int STAGES, int GROUPED>
__global__ void __launch_bounds__(192, 1)
k_gemm_tcp(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_u,
           const __grid_constant__ CUtensorMap map_x, TcpArgs p) {
  constexpr uint32_t B_BYTES = TN * BK * 2;
  constexpr uint32_t W_BYTES = A_BYTES * (1 + PAIR);
  constexpr uint32_t STAGE_BYTES = W_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = TN * (1 + PAIR);  // columns of one accumulator buffer
  constexpr uint32_t NCOLS = 2 * ACC_COLS;        // both buffers: 512 for TN = 256 or PAIR with TN = 128
  static_assert(NCOLS <= 512 && (NCOLS & (NCOLS - 1)) == 0 && NCOLS >= 32, "TMEM columns");

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * STAGE_BYTES;  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  const uint32_t bar_acc_full = bars + 16 * STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  uint8_t* gen = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 32);
  volatile int* cta_abort = (volatile int*)(gen + STAGES * STAGE_BYTES + 16 * STAGES + 36);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nkb = p.kb_total;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bars + 8 * s, 1);             // full[s]: one expect_tx covering every box of the stage
      mbar_init(bars + 8 * (STAGES + s), 1);  // empty[s]: one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);     // one tcgen05.commit
      mbar_init(bar_acc_empty + 8 * b, 128);  // every epilogue thread
    }
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
  const uint32_t tmem_base = *tmem_slot;

  // activations, the residual, the output (and the tile list) belong to the stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int total_tiles = (GROUPED ? *p.n_list : p.m_tiles) * p.n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileAt ta = tile_at<TN, GROUPED>(p, t);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (it >= STAGES) {
            ok = mbar_wait(bars + 8 * (STAGES + s), ((it / STAGES) & 1u) ^ 1u, cta_abort, p.err);
            if (!ok) break;
          }
          const uint32_t full = bars + 8 * s;
          const uint32_t a = base + s * STAGE_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_2d(a, &map_w, kb * BK, ta.wrow, full);
          if (PAIR) tma_load_2d(a + A_BYTES, GROUPED ? &map_u : &map_w, kb * BK, GROUPED ? ta.wrow : ta.wrow + p.row2_off, full);
          tma_load_2d(a + W_BYTES, &map_x, kb * BK, ta.m0, full);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(TN);
      uint32_t it = 0;
      int ti = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++ti) {
        const uint32_t buf = (uint32_t)ti & 1u;
        if (ti >= 2) {
          ok = mbar_wait(bar_acc_empty + 8 * buf, (((uint32_t)ti >> 1) & 1u) ^ 1u, cta_abort, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          ok = mbar_wait(bars + 8 * s, (it / STAGES) & 1u, cta_abort, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = base + s * STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t db = umma_desc(a + W_BYTES + kk * UMMA_K * 2);
            umma_bf16(acc, umma_desc(a + kk * UMMA_K * 2), db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            if (PAIR) umma_bf16(acc + TN, umma_desc(a + A_BYTES + kk * UMMA_K * 2), db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(bars + 8 * (STAGES + s));
        }
        if (ok) umma_commit(bar_acc_full + 8 * buf);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id mod 4)
    const int row = q * 32 + lane;
    int ti = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++ti) {
      const uint32_t buf = (uint32_t)ti & 1u;
      const TileAt ta = tile_at<TN, GROUPED>(p, t);
      const int m0 = ta.m0, m_end = ta.m_end;
      const int n = ta.n0 + row;
      ok = mbar_wait(bar_acc_full + 8 * buf, ((uint32_t)ti >> 1) & 1u, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        if (m0 + c0 >= m_end) break;
        uint32_t v[16];
        tmem_ld16(acc + (uint32_t)c0, v);
        if (PAIR) {
          uint32_t u[16];
          tmem_ld16(acc + (uint32_t)(TN + c0), u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c0 + j;
              if (m >= m_end) break;
              const float g = __uint_as_float(v[j]);
              const float h = (p.act == 0 ? silu_f(g) : gelu_f(g)) * __uint_as_float(u[j]);
              ((__nv_bfloat16*)p.out)[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(h);
            }
          }
        } else {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (n < p.N) {
            if (p.out_mode == 2) {
              // out may alias residual: all loads of the group before its stores
              float res[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c0 + j;
                res[j] = m < m_end ? p.residual[(int64_t)m * p.ldo + n] : 0.f;
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c0 + j;
                if (m < m_end) ((float*)p.out)[(int64_t)m * p.ldo + n] = __uint_as_float(v[j]) + res[j];
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c0 + j;
                if (m >= m_end) break;
                if (p.out_mode == 0) ((float*)p.out)[(int64_t)m * p.ldo + n] = __uint_as_float(v[j]);
                else ((__nv_bfloat16*)p.out)[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(__uint_as_float(v[j]));
              }
            }
          }
        }
      }
      // this half of TMEM may be overwritten once all four warps have read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(NCOLS) : "memory");
  }
}

template <int TN, int PAIR, int STAGES, int GROUPED>
int launch_tcp(cg_ctx* c, const CUtensorMap& mw, const CUtensorMap& mu, const CUtensorMap& mx, const TcpArgs& a, int ctas) {
  constexpr size_t smem = (size_t)STAGES * (A_BYTES * (1 + PAIR) + TN * BK * 2) + 1024 + 16 * STAGES + 64;
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_gemm_tcp<TN, PAIR, STAGES, GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  CG_CUDA(c, launch_kernel(c, k_gemm_tcp<TN, PAIR, STAGES, GROUPED>, dim3((unsigned)ctas), dim3(192), smem, 1, mw, mu, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

int sm_count(cg_ctx* c) {
  static int n = 0;
  if (!n) {
    cudaDeviceProp pr;
    n = cudaGetDeviceProperties(&pr, c->core->device) == cudaSuccess ? pr.multiProcessorCount : 148;
  }
  return n;
}

}  // namespace

bool gemm_tcp_wanted(int64_t M, int64_t N, int64_t K) {
  // enough 128 x 256 tiles that every SM gets at least two, and a k loop worth pipelining
  return M >= 512 && ((M + 255) / 256) * ((N + BM - 1) / BM) >= 200 && K >= 4 * BK;
}

int gemm_tcp(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, int64_t w_rows, void* out,
             int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K, int out_mode, int pair, int act) {
  if (M <= 0 || N <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp: k and leading dimensions must be multiples of 8, bases 16-byte aligned");
  if (M > 2147483647ll / 2 || N > 2147483647ll / 4) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp: problem too large");
  const int tn = pair ? 128 : 256;
  CUtensorMap mw, mx;
  CG_TRY(make_map(c, &mw, w, w_rows, K, ldw, BM));
  CG_TRY(make_map(c, &mx, x, M, K, ldx, tn));
  TcpArgs a;
  a.out = out; a.residual = residual; a.ldo = ldo;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.out_mode = pair ? 1 : out_mode;
  a.kb_total = (int)((K + BK - 1) / BK);
  a.m_tiles = (int)((M + tn - 1) / tn);
  a.n_tiles = (int)((N + BM - 1) / BM);
  a.row2_off = (int)N;
  a.act = act;
  a.tile_expert = a.tile_row0 = a.tile_rows = a.n_list = nullptr;
  a.w_rows = 0;
  a.err = c->core->dev_err;
  const int64_t tiles = (int64_t)a.m_tiles * a.n_tiles;
  if (tiles > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp: too many tiles");
  const int ctas = (int)std::min<int64_t>(tiles, sm_count(c));
  if (pair) return launch_tcp<128, 1, 4, 0>(c, mw, mw, mx, a, ctas);
  return launch_tcp<256, 0, 4, 0>(c, mw, mw, mx, a, ctas);
}

// Grouped (mixture-of-experts) form over a device-built list of 128-token tiles; see
// moe.cu.  w (and w_up when pair) are the experts' matrices stacked along the rows
// ([experts * N, K]); x holds the grouped activation rows; out rows follow x.
int gemm_tcp_grouped(cg_ctx* c, const __nv_bfloat16* x, int64_t x_rows, const __nv_bfloat16* w, const __nv_bfloat16* w_up,
                     int64_t experts, void* out, int64_t N, int64_t K, int pair, int act, const int32_t* tile_expert,
                     const int32_t* tile_row0, const int32_t* tile_rows, const int32_t* n_list, int64_t max_list) {
  if (x_rows <= 0 || N <= 0 || experts <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16) || (pair && ((uintptr_t)w_up % 16)))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp: k must be a multiple of 8, bases 16-byte aligned");
  CUtensorMap mw, mu, mx;
  CG_TRY(make_map(c, &mw, w, experts * N, K, K, BM));
  CG_TRY(make_map(c, &mu, pair ? w_up : w, experts * N, K, K, BM));
  CG_TRY(make_map(c, &mx, x, x_rows, K, K, 128));
  TcpArgs a;
  a.out = out; a.residual = nullptr; a.ldo = N;
  a.M = (int)x_rows; a.N = (int)N; a.K = (int)K;
  a.out_mode = pair ? 1 : 0;
  a.kb_total = (int)((K + BK - 1) / BK);
  a.m_tiles = 0;
  a.n_tiles = (int)((N + BM - 1) / BM);
  a.row2_off = 0;
  a.act = act;
  a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.tile_rows = tile_rows; a.n_list = n_list;
  a.w_rows = (int)N;
  a.err = c->core->dev_err;
  const int ctas = (int)std::min<int64_t>(max_list * a.n_tiles, sm_count(c));
  if (pair) return launch_tcp<128, 1, 4, 1>(c, mw, mu, mx, a, ctas);
  return launch_tcp<128, 0, 6, 1>(c, mw, mu, mx, a, ctas);
}

}  // namespace cg
