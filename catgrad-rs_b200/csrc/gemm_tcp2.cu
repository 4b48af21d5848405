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
//   warp 0            TMA producer (both CTAs, each into its own shared memory; the bytes of
//                     both are counted on rank 0's "stage full" barrier: the cta_group::2
//                     form of the tile load: every CTA fetches its own bytes)
//   warp 1            rank 0: issues the pair's MMAs once the pair's stage has landed;
//                     releases stages and publishes accumulators with tcgen05.commit to the
//                     barrier of each CTA in turn.  rank 1: idle after the TMEM allocation.
//   warps 2-9         epilogue of the CTA's own accumulator rows (two warps per TMEM lane
//                     quarter, each taking half of the tokens); one lane per warp tells rank 0
//                     that a buffer may be overwritten
//
// GLU form (gate/up of the FFN, catgrad-llm/src/models/llama.rs:27): every 32 A rows of a CTA
// -- the TMEM lanes one epilogue warp can read -- are 16 gate rows followed by the 16 matching
// up rows (one TMA box of a 4-d view of the stacked weight), so gate and up of a feature sit in lanes l
// and l + 16 of one warp and are swapped with a shuffle; the epilogue stores act(gate) * up in
// bf16.  The [M, 2F] intermediate never exists, as in the one-CTA kernel's PAIR form.
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
constexpr int P2_MAX_STAGES = 7;  // 7 x 32 KB + barriers fit the 227 KB a CTA may have
constexpr uint32_t P2_B_BYTES = P2_TOK_CTA * BK * 2;
constexpr uint32_t P2_STAGE_BYTES = A_BYTES + P2_B_BYTES;  // 32 KB
constexpr uint32_t P2_NCOLS = 512;                         // two accumulator buffers of 256 columns

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
  int stages;    // ring slots in use (<= P2_MAX_STAGES)
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
// The same for a 4-d tensor map (the interleaved gate/up view of make_map_glu).
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// TMA tile load of a CTA pair: the bytes land in THIS CTA's shared memory and are counted on a
// barrier that may live in the peer CTA (given by its shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
// 32 consecutive TMEM columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
        "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

template <int GLU>
__global__ void __launch_bounds__(320, 1)
k_gemm_tcp2(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Tcp2Args p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  // barriers: full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t P2_STAGES = (uint32_t)p.stages;
  const uint32_t bars = base + P2_MAX_STAGES * P2_STAGE_BYTES;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * P2_MAX_STAGES;
  const uint32_t bar_acc_full = bars + 16 * P2_MAX_STAGES, bar_acc_empty = bar_acc_full + 16;
  uint8_t* gen = smem_raw + (base - raw);
  uint8_t* tail = gen + P2_MAX_STAGES * P2_STAGE_BYTES + 16 * P2_MAX_STAGES + 32;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)tail;
  volatile int* cta_abort = (volatile int*)(tail + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int nkb = p.kb_total;

  if (tid == 0) {
    for (int s = 0; s < P2_MAX_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);       // rank 0 only: one expect_tx covering the boxes of both CTAs' stage
      mbar_init(bar_empty + 8 * s, 1);      // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);   // one tcgen05.commit
      mbar_init(bar_acc_empty + 8 * b, 16);  // rank 0 only: one lane of each epilogue warp of both CTAs
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
      const uint32_t full0 = map_to_rank(bar_full, 0);
      uint32_t s = 0, ph = 0;  // ring slot and the parity of its use (no runtime division in the loop)
      bool first_lap = true;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += pairs) {
        const int m0 = (t % p.m_tiles) * P2_TOK + (int)rank * P2_TOK_CTA;
        const int n0 = (t / p.m_tiles) * (GLU ? P2_ROWS / 2 : P2_ROWS) + (int)rank * (GLU ? 64 : 128);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!first_lap) {
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, cta_abort, p.err);
            if (!ok) break;
          }
          // both CTAs' bytes are counted on rank 0's barrier, which expects the pair's stage
          const uint32_t full = full0 + 8 * s;
          const uint32_t a = base + s * P2_STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * P2_STAGE_BYTES);
          if (GLU) {
            // one box of the 4-d view: per 32 A rows (one epilogue warp's TMEM lanes) 16 gate
            // rows, then their up rows
            tma_load_4d_pair(a, &map_w, kb * BK, 0, 0, n0 >> 4, full);
          } else {
            tma_load_2d_pair(a, &map_w, kb * BK, n0, full);
          }
          tma_load_2d_pair(a + A_BYTES, &map_x, kb * BK, m0, full);
          if (++s == P2_STAGES) { s = 0; ph ^= 1u; first_lap = false; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_m256(P2_TOK);
      uint32_t empty_at[2], acc_full_at[2];
      for (uint32_t r = 0; r < 2; ++r) {
        empty_at[r] = map_to_rank(bar_empty, r);
        acc_full_at[r] = map_to_rank(bar_acc_full, r);
      }
      uint32_t s = 0, par = 0;
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
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(bar_full + 8 * s, par, cta_abort, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = base + s * P2_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma2_bf16(acc, umma_desc(a + kk * UMMA_K * 2), umma_desc(a + A_BYTES + kk * UMMA_K * 2), idesc,
                       (kb > 0 || kk > 0) ? 1u : 0u);
          umma2_commit(empty_at[0] + 8 * s);
          umma2_commit(empty_at[1] + 8 * s);
          if (++s == P2_STAGES) { s = 0; par ^= 1u; }
        }
        if (ok) {
          umma2_commit(acc_full_at[0] + 8 * buf);
          umma2_commit(acc_full_at[1] + 8 * buf);
        }
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id mod 4)
    const int col0 = warp >= 6 ? P2_TOK / 2 : 0;  // two warps per lane quarter: each takes half of the tokens
    const int row = q * 32 + lane;
    const uint32_t acc_empty_at = map_to_rank(bar_acc_empty, 0);
    int ti = 0;
    bool ok = true;
    for (int t = pair; t < total_tiles && ok; t += pairs, ++ti) {
      const uint32_t buf = (uint32_t)ti & 1u;
      const int m0 = (t % p.m_tiles) * P2_TOK, m_end = p.M;
      ok = mbar_wait(bar_acc_full + 8 * buf, ((uint32_t)ti >> 1) & 1u, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * P2_TOK + ((uint32_t)(q * 32) << 16);
      // 32 tokens per round; the TMEM load of the next round flies while this one is finished.
      // Rounds run as a rolled loop of two (the two register buffers): unrolled over the whole
      // tile the epilogue would push the MMA and TMA loops out of the instruction cache.
      uint32_t va[32], vb[32];
      tmem_ld32(acc + (uint32_t)col0, va);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (GLU) {
        // lanes 0..15 of a warp hold gate, lanes 16..31 up, of features n_base + 16 q + (lane mod
        // 16): the halves swap what the other needs with one shuffle per value.  Of every 32
        // tokens the gate lanes finish the first 16 and the up lanes the last 16.
        const bool is_up = lane >= 16;
        const int n = (t / p.m_tiles) * (P2_ROWS / 2) + (int)rank * 64 + q * 16 + (lane & 15);
        __nv_bfloat16* const dst = (__nv_bfloat16*)p.out + n;
        auto round = [&](const uint32_t* cur, uint32_t* nxt, int c0) {
          if (c0 + 32 < col0 + P2_TOK / 2) tmem_ld32(acc + (uint32_t)(c0 + 32), nxt);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t send = is_up ? cur[j] : cur[16 + j];
            const float other = __uint_as_float(__shfl_xor_sync(0xffffffffu, send, 16));
            const float g = is_up ? other : __uint_as_float(cur[j]);
            const float u = is_up ? __uint_as_float(cur[16 + j]) : other;
            const int m = m0 + c0 + (is_up ? 16 : 0) + j;
            if (n < p.N && m < m_end) {
              const float h = (p.act == 0 ? silu_fast(g) : gelu_fast(g)) * u;
              dst[(int64_t)m * p.ldo] = __float2bfloat16_rn(h);
            }
          }
          if (c0 + 32 < col0 + P2_TOK / 2) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        };
#pragma unroll 1
        for (int c0 = col0; c0 < col0 + P2_TOK / 2; c0 += 64) {
          if (m0 + c0 >= m_end) break;  // uniform over the warp
          round(va, vb, c0);
          round(vb, va, c0 + 32);
        }
      } else {
        const int n = (t / p.m_tiles) * P2_ROWS + (int)rank * 128 + row;
        const bool live = n < p.N;
        auto round = [&](const uint32_t* cur, uint32_t* nxt, int c0) {
          if (c0 + 32 < col0 + P2_TOK / 2) tmem_ld32(acc + (uint32_t)(c0 + 32), nxt);
          if (live) {
            if (p.out_mode == 2) {
              // out may alias residual: all loads of the round before its stores (and all 32 in
              // flight together)
              float res[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int m = m0 + c0 + j;
                res[j] = m < m_end ? p.residual[(int64_t)m * p.ldo + n] : 0.f;
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int m = m0 + c0 + j;
                if (m < m_end) ((float*)p.out)[(int64_t)m * p.ldo + n] = __uint_as_float(cur[j]) + res[j];
              }
            } else if (p.out_mode == 0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int m = m0 + c0 + j;
                if (m < m_end) ((float*)p.out)[(int64_t)m * p.ldo + n] = __uint_as_float(cur[j]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int m = m0 + c0 + j;
                if (m < m_end) ((__nv_bfloat16*)p.out)[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(__uint_as_float(cur[j]));
              }
            }
          }
          if (c0 + 32 < col0 + P2_TOK / 2) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        };
#pragma unroll 1
        for (int c0 = col0; c0 < col0 + P2_TOK / 2; c0 += 64) {
          if (m0 + c0 >= m_end) break;
          round(va, vb, c0);
          round(vb, va, c0 + 32);
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

// The stacked gate/up weight [2F, K] (gate rows first) as a 4-d tensor {K, 16, 2, F / 16}: a box
// of {64, 16, 2, 4} lands in shared memory as 4 x (16 gate rows, their 16 up rows) of 64 k
// values each -- the 128-row A tile of the GLU form in one request.  F must be a multiple of 16.
int make_map_glu(cg_ctx* c, CUtensorMap* map, const void* w, int64_t F, int64_t K, int64_t ldw) {
  if (!c->encode_tiled) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return fail(c, CG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    c->encode_tiled = fn;
  }
  cuuint64_t gdim[4] = {(cuuint64_t)K, 16, 2, (cuuint64_t)(F / 16)};
  cuuint64_t gstr[3] = {(cuuint64_t)ldw * 2, (cuuint64_t)F * ldw * 2, (cuuint64_t)16 * ldw * 2};
  cuuint32_t box[4] = {(cuuint32_t)BK, 16, 2, 4};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = ((EncodeTiledFn)c->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(w), gdim, gstr, box,
                                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, CG_ERR_CUDA, "cuTensorMapEncodeTiled (4-d) failed with code " + std::to_string((int)r));
  return CG_OK;
}

constexpr size_t P2_SMEM = (size_t)P2_MAX_STAGES * P2_STAGE_BYTES + 1024 + 16 * P2_MAX_STAGES + 32 + 16 + 64;

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
  CG_CUDA(c, launch_kernel(c, k_gemm_tcp2<GLU>, dim3(2u * (unsigned)pairs, 1, 1), dim3(320), P2_SMEM, -2, mw, mx, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

bool gemm_tcp2_supported(int64_t N, int glu) { return !glu || N % 16 == 0; }

bool gemm_tcp2_wanted(int64_t M, int64_t N, int64_t K, int glu) {
  if (!gemm_tcp2_supported(N, glu)) return false;
  // enough 256 x 256 tiles for one and a half per pair of SMs, and a k loop worth pipelining
  // (measured on the Llama-3.2-1B widths at 4096 tokens: with every projection on pairs the
  // prefill takes 8.33 ms, with only the gate/up form 8.92 ms, with none 9.46 ms)
  const int64_t rows = glu ? 2 * N : N;
  return M >= 1024 && ((M + 255) / 256) * ((rows + 255) / 256) >= 111 && K >= 8 * BK;
}

int gemm_tcp2(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, int64_t w_rows, void* out,
              int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K, int out_mode, int glu, int act) {
  if (M <= 0 || N <= 0) return CG_OK;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: k and leading dimensions must be multiples of 8, bases 16-byte aligned");
  if (M > 2147483647ll / 2 || N > 2147483647ll / 4) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: problem too large");
  CUtensorMap mw, mx;
  if (glu) {
    if (N % 16 || w_rows != 2 * N) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: the gate/up form wants F a multiple of 16");
    CG_TRY(make_map_glu(c, &mw, w, N, K, ldw));
  } else {
    CG_TRY(make_map(c, &mw, w, w_rows, K, ldw, 128));
  }
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
  a.stages = P2_MAX_STAGES;  // (six stages measured the same as seven)
  a.err = c->core->dev_err;
  const int64_t tiles = (int64_t)a.m_tiles * a.n_tiles;
  if (tiles > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "gemm_tcp2: too many tiles");
  // (an attribute query, not cudaGetDeviceProperties: that call takes milliseconds)
  int sms = 148;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->core->device) != cudaSuccess || sms < 2) sms = 148;
  const int pairs = (int)std::min<int64_t>(tiles, sms / 2);
  if (glu) return launch_tcp2<1>(c, mw, mx, a, pairs);
  return launch_tcp2<0>(c, mw, mx, a, pairs);
}

}  // namespace cg
