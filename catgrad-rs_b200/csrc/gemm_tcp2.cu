// gemm_tcp2.cu — the persistent many-token GEMM on CTA pairs: y[M,N] = x[M,K] w[N,K]^T with
// tcgen05.mma.cta_group::2.
//
// Why pairs: the one-CTA kernel (gemm_tcp.cu) loads 48 KB per 64-wide k block for its
// 128 x 256 tile -- a tile of W and the whole activation tile -- and its tensor pipe waits on
// the SM's L2 read path.  Two CTAs of a cluster (the two SMs of a TPC) that work on one
// 256 (rows of W) x 256 (tokens) tile each load their own 128 rows of W and only HALF of the
// activation tile, 32 KB per k block for the same math per SM; the MMA unit of each SM reads
// the other half out of the peer's shared memory.
//
//   CTA r of a pair   A operand: W rows n0 + 128 r ... (its own shared memory)
//                     B operand: tokens m0 + 128 r ... (each CTA holds half of the N side)
//                     accumulator (its own TMEM): lanes = its 128 W rows, columns = all 256
//                     tokens, double-buffered (2 x 256 columns)
//   warp 0            TMA producer (both CTAs, each for its own shared memory; plain loads
//                     that complete on a barrier of the same CTA)
//   warp 1            rank 0: issues the pair's MMAs once its own and the peer's stage have
//                     landed; releases stages and publishes accumulators with tcgen05.commit
//                     to the barrier of each CTA in turn.  rank 1: relays "my stage has
//                     landed" to rank 0 (mbarrier arrive with cluster scope).
//   warps 2-5         epilogue of the CTA's own accumulator rows; one lane per warp tells
//                     rank 0 that a buffer may be overwritten
//
// GLU form (gate/up of the FFN, catgrad-llm/src/models/llama.rs:27): the 128 A rows of a CTA
// are 64 gate rows followed by the 64 matching up rows (two TMA boxes), so gate and up of a
// feature sit in lanes l and l + 64 of the same accumulator columns; the epilogue warps swap
// halves through shared memory and store act(gate) * up in bf16.  The [M, 2F] intermediate
// never exists, as in the one-CTA kernel's PAIR form.
//
// Every wait is bounded (tc_common.cuh); after an expiry all roles of both CTAs leave their
// loops, meet at the closing cluster barrier, free TMEM and return.
#include <algorithm>

#include "act.cuh"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

constexpr int P2_TOK = 256;      // tokens per pair tile (MMA N)
constexpr int P2_TOK_CTA = 128;  // token rows one CTA loads
constexpr int P2_ROWS = 256;     // W rows per pair tile (MMA M), 128 per CTA
constexpr int P2_STAGES = 6;
constexpr uint32_t P2_B_BYTES = P2_TOK_CTA * BK * 2;
constexpr uint32_t P2_STAGE_BYTES = A_BYTES + P2_B_BYTES;  // 32 KB
constexpr uint32_t P2_NCOLS = 512;                         // two accumulator buffers of 256 columns
constexpr int P2_XCH_LD = 9;                               // padded row of the gate/up exchange area

struct Tcp2Args {
  void* out;
  const float* residual;
  int64_t ldo;
  int M, N, K;
  int out_mode;  // 0 f32, 1 bf16, 2 f32 + residual (residual may alias out)
  int kb_total;
  int m_tiles, n_tiles;
  int row2_off;  // GLU: rows between a gate row and its up row
  int act;       // GLU: 0 silu, 1 tanh-gelu
  int32_t* err;
};

// Instruction descriptor: bf16 x bf16 -> f32, both operands k-major, M = 256 over the pair, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_m256(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrival on one barrier (given by its shared::cluster address) once the pair's MMAs issued so far are done
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int GLU>
__global__ void __launch_bounds__(192, 1)
k_gemm_tcp2(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Tcp2Args p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  // barriers: full[S], peer_full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t bars = base + P2_STAGES * P2_STAGE_BYTES;
  const uint32_t bar_full = bars, bar_peer_full = bars + 8 * P2_STAGES, bar_empty = bars + 16 * P2_STAGES;
  const uint32_t bar_acc_full = bars + 24 * P2_STAGES, bar_acc_empty = bar_acc_full + 16;
  uint8_t* gen = smem_raw + (base - raw);
  uint8_t* tail = gen + P2_STAGES * P2_STAGE_BYTES + 24 * P2_STAGES + 32;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)tail;
  volatile int* cta_abort = (volatile int*)(tail + 4);
  float* xch = (float*)(tail + 16);  // GLU: [2 buffers][2 halves][64 lanes][P2_XCH_LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int nkb = p.kb_total;

  if (tid == 0) {
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);       // one expect_tx covering the boxes of the stage
      mbar_init(bar_peer_full + 8 * s, 1);  // rank 0 only: the peer's relay
      mbar_init(bar_empty + 8 * s, 1);      // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);   // one tcgen05.commit
      mbar_init(bar_acc_empty + 8 * b, 8);  // rank 0 only: one lane of each epilogue warp of both CTAs
    }
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // one warp of each CTA of the pair takes part in the pair's allocation
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"(P2_NCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // activations, the residual and the output belong to the stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int total_tiles = p.m_tiles * p.n_tiles;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += pairs) {
        const int m0 = (t % p.m_tiles) * P2_TOK + (int)rank * P2_TOK_CTA;
        const int n0 = (t / p.m_tiles) * (GLU ? P2_ROWS / 2 : P2_ROWS) + (int)rank * (GLU ? 64 : 128);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % P2_STAGES;
          if (it >= P2_STAGES) {
            ok = mbar_wait_cluster(bar_empty + 8 * s, ((it / P2_STAGES) & 1u) ^ 1u, cta_abort, p.err);
            if (!ok) break;
          }
          const uint32_t full = bar_full + 8 * s;
          const uint32_t a = base + s * P2_STAGE_BYTES;
          mbar_expect_tx(full, P2_STAGE_BYTES);
          if (GLU) {
            tma_load_2d(a, &map_w, kb * BK, n0, full);                             // 64 gate rows
            tma_load_2d(a + A_BYTES / 2, &map_w, kb * BK, n0 + p.row2_off, full);  // their up rows
          } else {
            tma_load_2d(a, &map_w, kb * BK, n0, full);
          }
          tma_load_2d(a + A_BYTES, &map_x, kb * BK, m0, full);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 1) {
      // relay: my stage has landed -> rank 0's peer_full
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += pairs) {
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % P2_STAGES;
          ok = mbar_wait(bar_full + 8 * s, (it / P2_STAGES) & 1u, cta_abort, p.err);
          if (!ok) break;
          mbar_arrive_remote(bar_peer_full + 8 * s, 0);
        }
      }
    } else if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_m256(P2_TOK);
      uint32_t empty_at[2], acc_full_at[2];
      for (uint32_t r = 0; r < 2; ++r) {
        empty_at[r] = map_to_rank(bar_empty, r);
        acc_full_at[r] = map_to_rank(bar_acc_full, r);
      }
      uint32_t it = 0;
      int ti = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += pairs, ++ti) {
        const uint32_t buf = (uint32_t)ti & 1u;
        if (ti >= 2) {
          ok = mbar_wait_cluster(bar_acc_empty + 8 * buf, (((uint32_t)ti >> 1) & 1u) ^ 1u, cta_abort, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + buf * P2_TOK;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % P2_STAGES;
          const uint32_t par = (it / P2_STAGES) & 1u;
          ok = mbar_wait(bar_full + 8 * s, par, cta_abort, p.err) && mbar_wait_cluster(bar_peer_full + 8 * s, par, cta_abort, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = base + s * P2_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma2_bf16(acc, umma_desc(a + kk * UMMA_K * 2), umma_desc(a + A_BYTES + kk * UMMA_K * 2), idesc,
                       (kb > 0 || kk > 0) ? 1u : 0u);
          umma2_commit(empty_at[0] + 8 * s);
          umma2_commit(empty_at[1] + 8 * s);
        }
        if (ok) {
          umma2_commit(acc_full_at[0] + 8 * buf);
          umma2_commit(acc_full_at[1] + 8 * buf);
        }
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id mod 4)
    const int row = q * 32 + lane;
    const uint32_t acc_empty_at = map_to_rank(bar_acc_empty, 0);
    int ti = 0;
    int xb = 0;  // exchange buffer of the next chunk: alternates over all chunks of all tiles
    bool ok = true;
    for (int t = pair; t < total_tiles && ok; t += pairs, ++ti) {
      const uint32_t buf = (uint32_t)ti & 1u;
      const int m0 = (t % p.m_tiles) * P2_TOK, m_end = p.M;
      ok = mbar_wait_cluster(bar_acc_full + 8 * buf, ((uint32_t)ti >> 1) & 1u, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * P2_TOK + ((uint32_t)(q * 32) << 16);
      if (GLU) {
        // lanes 0..63 hold gate, 64..127 up, of features n_base + (lane mod 64).  Per 16 tokens
        // the gate warps finish tokens 0..7 and the up warps tokens 8..15, after handing the
        // other half of what they hold to the warp 64 lanes away.
        const int n = (t / p.m_tiles) * (P2_ROWS / 2) + (int)rank * 64 + (row & 63);
        const bool is_up = row >= 64;
#pragma unroll 1
        for (int c0 = 0; c0 < P2_TOK; c0 += 16, xb ^= 1) {
          if (m0 + c0 >= m_end) break;  // uniform over the CTA
          uint32_t v[16];
          tmem_ld16(acc + (uint32_t)c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          float* mine = xch + ((xb * 2 + (is_up ? 1 : 0)) * 64 + (row & 63)) * P2_XCH_LD;
          const float* theirs = xch + ((xb * 2 + (is_up ? 0 : 1)) * 64 + (row & 63)) * P2_XCH_LD;
#pragma unroll
          for (int j = 0; j < 8; ++j) mine[j] = __uint_as_float(is_up ? v[j] : v[8 + j]);
          epi_bar();
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int m = m0 + c0 + (is_up ? 8 : 0) + j;
              if (m >= m_end) break;
              const float g = is_up ? theirs[j] : __uint_as_float(v[j]);
              const float u = is_up ? __uint_as_float(v[8 + j]) : theirs[j];
              const float h = (p.act == 0 ? silu_f(g) : gelu_f(g)) * u;
              ((__nv_bfloat16*)p.out)[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(h);
            }
          }
          // the other buffer is written next: whoever read it last did so before this chunk's
          // barrier (chunks alternate buffers across tile boundaries too)
        }
      } else {
        const int n = (t / p.m_tiles) * P2_ROWS + (int)rank * 128 + row;
#pragma unroll 1
        for (int c0 = 0; c0 < P2_TOK; c0 += 16) {
          if (m0 + c0 >= m_end) break;
          uint32_t v[16];
          tmem_ld16(acc + (uint32_t)c0, v);
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
      // this buffer may be overwritten once the four warps of both CTAs have read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(acc_empty_at + 8 * buf) : "memory");
    }
  }

  // nobody leaves, and no TMEM is freed, while the peer may still read this CTA's shared
  // memory, arrive on its barriers or run MMAs into its TMEM
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P2_NCOLS) : "memory");
  }
}

constexpr size_t P2_SMEM = (size_t)P2_STAGES * P2_STAGE_BYTES + 1024 + 24 * P2_STAGES + 32 + 16 + 2 * 2 * 64 * P2_XCH_LD * 4 + 64;

template <int GLU>
int launch_tcp2(cg_ctx* c, const CUtensorMap& mw, const CUtensorMap& mx, const Tcp2Args& a, int pairs) {
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_gemm_tcp2<GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM));
    configured = true;
  }
  // clusters of (2, 1, 1): a kernel that uses cta_group::2 is refused at launch with any other
  // pairing ("cluster misconfiguration" for clusters of (1, 1, 2)).  blockIdx.x / 2 is the pair.
  CG_CUDA(c, launch_kernel(c, k_gemm_tcp2<GLU>, dim3(2u * (unsigned)pairs, 1, 1), dim3(192), P2_SMEM, -2, mw, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

bool gemm_tcp2_wanted(int64_t M, int64_t N, int64_t K, int glu) {
  // at least two 256 x 256 tiles for every pair of SMs, and a k loop worth pipelining
  const int64_t rows = glu ? 2 * N : N;
  return M >= 1024 && ((M + 255) / 256) * ((rows + 255) / 256) >= 148 && K >= 8 * BK;
}

int gemm_tcp2(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, int64_t w_rows, void* out,
              int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K, int out_mode, int glu, int act) {
  if (M <= 0 || N <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: k and leading dimensions must be multiples of 8, bases 16-byte aligned");
  if (M > 2147483647ll / 2 || N > 2147483647ll / 4) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: problem too large");
  CUtensorMap mw, mx;
  CG_TRY(make_map(c, &mw, w, w_rows, K, ldw, glu ? 64 : 128));
  CG_TRY(make_map(c, &mx, x, M, K, ldx, P2_TOK_CTA));
  Tcp2Args a;
  a.out = out; a.residual = residual; a.ldo = ldo;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.out_mode = glu ? 1 : out_mode;
  a.kb_total = (int)((K + BK - 1) / BK);
  a.m_tiles = (int)((M + P2_TOK - 1) / P2_TOK);
  a.n_tiles = (int)((N + (glu ? 127 : 255)) / (glu ? 128 : 256));
  a.row2_off = (int)N;
  a.act = act;
  a.err = c->core->dev_err;
  const int64_t tiles = (int64_t)a.m_tiles * a.n_tiles;
  if (tiles > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: too many tiles");
  int sms = 148;
  {
    cudaDeviceProp pr;
    if (cudaGetDeviceProperties(&pr, c->core->device) == cudaSuccess) sms = pr.multiProcessorCount;
  }
  const int pairs = (int)std::min<int64_t>(tiles, sms / 2);
  if (glu) return launch_tcp2<1>(c, mw, mx, a, pairs);
  return launch_tcp2<0>(c, mw, mx, a, pairs);
}

}  // namespace cg
