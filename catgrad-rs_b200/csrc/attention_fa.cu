// attention_fa.cu — causal prefill attention on the Blackwell tensor cores (tcgen05 + TMEM),
// for head sizes 64 and 128 without soft-cap or window.
//
// Same mathematics as attention.cu (catgrad-llm/src/models/llama.rs:97-108 after repeat_kv,
// catgrad-llm/src/helpers.rs:147-161, as an online-softmax pass over key tiles); what changes
// is where the two matrix products run:
//
//   warp 0      TMA: the 128-query tile once, then 128-key K and V tiles through two
//               shared-memory buffers each
//   warp 1      one lane issues S = Q K^T (128 x 128, f32 in TMEM, two S buffers so the next
//               tile's scores are computed while this tile's softmax runs) and O_t = P V
//               (128 x D, f32 in TMEM)
//   warps 2-5   one thread per query row (TMEM lane = row, so row maxima and sums need no
//               shuffles): read the score row from TMEM, mask, exponentiate, write P as bf16
//               into shared memory in the 128-byte-swizzled k-major layout the MMA reads,
//               then fold O_t into the row's running output kept in registers
//
// V is consumed as it lies in the cache ([keys, D], D contiguous): for P V it is the MMA's B
// operand with the "MN-major" layout bit, i.e. no transposed copy of V exists anywhere.
//
// Every mbarrier wait is bounded; on expiry the kernel raises the context's error word, all
// roles leave their loops, TMEM is freed and the kernel returns.
#include <algorithm>

#include "kernels.h"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

constexpr int FA_BQ = 128;

struct FaArgs {
  __nv_bfloat16* out;  // [B * S, nh D]
  int64_t S, pos0, Tmax;
  int nh, nkv;
  float scale_log2e;   // 1 / sqrt(D) * log2(e)
  int32_t* err;
};

// B operand stored [k rows][n contiguous] ("MN-major") in 128-byte-swizzled boxes of
// [rows, 64 elements]: 64-element chunks along n are `chunk_bytes` apart, groups of 8 k rows
// 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t saddr, uint32_t chunk_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((chunk_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset: next 64-element chunk along n
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: next group of 8 k rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}

template <int D, int FA_BK>
__global__ void __launch_bounds__(192, FA_BK == 64 ? 2 : 1)
k_attn_fa(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
          const __grid_constant__ CUtensorMap map_v, FaArgs p) {
  constexpr int SUB = D / 64;                       // 64-wide sub-tiles along the head dimension
  constexpr uint32_t BOX = 128 * 128;               // bytes of one [128 rows, 64 bf16] box (Q, P)
  constexpr uint32_t KBOX = FA_BK * 128;            // bytes of one [FA_BK keys, 64 bf16] box (K, V)
  constexpr uint32_t Q_BYTES = SUB * BOX, KV_BYTES = SUB * KBOX, P_BYTES = (FA_BK / 64) * BOX;
  constexpr uint32_t S_COLS = FA_BK;                // one score buffer
  constexpr uint32_t O_COL = 2 * S_COLS;            // O_t after the two score buffers
  constexpr uint32_t NCOLS = 2 * S_COLS + D <= 256 ? 256 : 512;  // two CTAs per SM share 512 columns

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  if (FA_BK == 64 && base != raw) {
    // the 64-key variant is sized without alignment slack (two CTAs must fit one SM)
    if (threadIdx.x == 0) *p.err = DEV_TIMEOUT;
    return;
  }
  const uint32_t sq = base, sk = sq + Q_BYTES, sv = sk + 2 * KV_BYTES, sp = sv + 2 * KV_BYTES;
  const uint32_t bars = sp + P_BYTES;
  uint8_t* gen = smem_raw + (base - raw);
  // barriers (8 bytes each)
  const uint32_t b_q_full = bars, b_k_full = bars + 8, b_v_full = bars + 24, b_k_empty = bars + 40, b_v_empty = bars + 56,
                 b_s_full = bars + 72, b_s_empty = bars + 88, b_p_full = bars + 104, b_p_empty = bars + 112,
                 b_o_full = bars + 120, b_o_empty = bars + 128;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen + (bars - base) + 144);
  volatile int* cta_abort = (volatile int*)(gen + (bars - base) + 148);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;  // longest tiles first
  const int64_t b = blockIdx.z;
  const int kvh = h / (p.nh / p.nkv);
  const int64_t q0 = (int64_t)qt * FA_BQ;
  const int64_t last_q = p.pos0 + std::min<int64_t>(p.S, q0 + FA_BQ) - 1;
  const int nt = (int)(last_q / FA_BK) + 1;  // key tiles 0 .. nt-1

  if (tid == 0) {
    mbar_init(b_q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(b_k_full + 8 * i, 1);
      mbar_init(b_v_full + 8 * i, 1);
      mbar_init(b_k_empty + 8 * i, 1);
      mbar_init(b_v_empty + 8 * i, 1);
      mbar_init(b_s_full + 8 * i, 1);
      mbar_init(b_s_empty + 8 * i, 128);
    }
    mbar_init(b_p_full, 128);
    mbar_init(b_p_empty, 1);
    mbar_init(b_o_full, 1);
    mbar_init(b_o_empty, 128);
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

  // q and the cache are written by the preceding kernels
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      const int qrow = (int)(b * p.S + q0);
      mbar_expect_tx(b_q_full, Q_BYTES);
      for (int s = 0; s < SUB; ++s) tma_load_2d(sq + s * BOX, &map_q, h * D + s * 64, qrow, b_q_full);
      const int64_t kvrow0 = (b * p.nkv + kvh) * p.Tmax;
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        const uint32_t buf = (uint32_t)j & 1u, ph = ((uint32_t)j >> 1) & 1u;
        const int row = (int)(kvrow0 + (int64_t)j * FA_BK);
        if (j >= 2) {
          ok = mbar_wait(b_k_empty + 8 * buf, ph ^ 1u, cta_abort, p.err);
          if (!ok) break;
        }
        mbar_expect_tx(b_k_full + 8 * buf, KV_BYTES);
        for (int s = 0; s < SUB; ++s) tma_load_2d(sk + buf * KV_BYTES + s * KBOX, &map_k, s * 64, row, b_k_full + 8 * buf);
        if (j >= 2) {
          ok = mbar_wait(b_v_empty + 8 * buf, ph ^ 1u, cta_abort, p.err);
          if (!ok) break;
        }
        mbar_expect_tx(b_v_full + 8 * buf, KV_BYTES);
        for (int s = 0; s < SUB; ++s) tma_load_2d(sv + buf * KV_BYTES + s * KBOX, &map_v, s * 64, row, b_v_full + 8 * buf);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(FA_BK);              // 128 x FA_BK, both operands k-major
      constexpr uint32_t idesc_o = umma_idesc(D) | (1u << 16);     // 128 x D, B operand MN-major
      bool ok = mbar_wait(b_q_full, 0, cta_abort, p.err);
      // S_j = Q K_j^T into score buffer j & 1
      auto issue_qk = [&](int j) {
        const uint32_t buf = (uint32_t)j & 1u, ph = ((uint32_t)j >> 1) & 1u;
        if (!mbar_wait(b_k_full + 8 * buf, ph, cta_abort, p.err)) return false;
        if (j >= 2 && !mbar_wait(b_s_empty + 8 * buf, ph ^ 1u, cta_abort, p.err)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < D / UMMA_K; ++kk) {
          const uint32_t offq = (uint32_t)(kk / 4) * BOX + (uint32_t)(kk % 4) * 32u;
          const uint32_t offk = (uint32_t)(kk / 4) * KBOX + (uint32_t)(kk % 4) * 32u;
          umma_bf16(tmem_base + buf * S_COLS, umma_desc(sq + offq), umma_desc(sk + buf * KV_BYTES + offk), idesc_s,
                    kk > 0 ? 1u : 0u);
        }
        umma_commit(b_s_full + 8 * buf);
        umma_commit(b_k_empty + 8 * buf);
        return true;
      };
      // O_t = P_j V_j
      auto issue_pv = [&](int j) {
        const uint32_t buf = (uint32_t)j & 1u, ph = ((uint32_t)j >> 1) & 1u;
        if (!mbar_wait(b_p_full, (uint32_t)j & 1u, cta_abort, p.err)) return false;
        if (!mbar_wait(b_v_full + 8 * buf, ph, cta_abort, p.err)) return false;
        if (j >= 1 && !mbar_wait(b_o_empty, ((uint32_t)j & 1u) ^ 1u, cta_abort, p.err)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < FA_BK / UMMA_K; ++kk) {
          const uint64_t da = umma_desc(sp + (uint32_t)(kk / 4) * BOX + (uint32_t)(kk % 4) * 32u);
          const uint64_t db = umma_desc_mn(sv + buf * KV_BYTES + (uint32_t)kk * (UMMA_K * 128u), KBOX);
          umma_bf16(tmem_base + O_COL, da, db, idesc_o, kk > 0 ? 1u : 0u);
        }
        umma_commit(b_o_full);
        umma_commit(b_v_empty + 8 * buf);
        umma_commit(b_p_empty);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nt && ok; ++j) {
        if (j + 1 < nt) ok = issue_qk(j + 1);
        if (ok) ok = issue_pv(j);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row of this thread = TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const int64_t qi = q0 + r;
    const int64_t qpos = p.pos0 + qi;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt && ok; ++j) {
      const uint32_t buf = (uint32_t)j & 1u, ph = ((uint32_t)j >> 1) & 1u;
      ok = mbar_wait(b_s_full + 8 * buf, ph, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t k0 = (int64_t)j * FA_BK;
      const bool diag = k0 + FA_BK - 1 > p.pos0 + q0;  // some key of the tile may be masked for some row
      // pass 1: row maximum of the visible scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BK; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(lane_base + buf * S_COLS + (uint32_t)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float s = __uint_as_float(v[i]);
          mx = (!diag || k0 + c0 + i <= qpos) ? fmaxf(mx, s) : mx;
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f((m - m_safe) * p.scale_log2e);  // 0 while m is -inf
      // the previous tile's P must have been consumed before it is overwritten
      if (j >= 1) {
        ok = mbar_wait(b_p_empty, ((uint32_t)j & 1u) ^ 1u, cta_abort, p.err);
        if (!ok) break;
      }
      // pass 2: p = exp2((s - m) * scale * log2 e), row sum, bf16 P into the swizzled tile
      float ls = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BK; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(lane_base + buf * S_COLS + (uint32_t)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float e0 = exp2f((__uint_as_float(v[i]) - m_safe) * p.scale_log2e);
          float e1 = exp2f((__uint_as_float(v[i + 1]) - m_safe) * p.scale_log2e);
          if (diag) {
            e0 = k0 + c0 + i <= qpos ? e0 : 0.f;
            e1 = k0 + c0 + i + 1 <= qpos ? e1 : 0.f;
          }
          // the sum uses the rounded values the MMA will see
          const __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
          ls += __low2float(pr) + __high2float(pr);
          pk[i / 2] = *(const uint32_t*)&pr;
        }
        // two 16-byte chunks of row r: chunk index ch = c0 / 8 (+1); sub-tile ch / 8, position (ch % 8) ^ (r % 8)
        const int ch = c0 / 8;
        const uint32_t rowb = sp + (uint32_t)(ch / 8) * BOX + (uint32_t)r * 128u;
        const uint32_t a0 = rowb + (uint32_t)(((ch % 8) ^ (r & 7)) * 16);
        const uint32_t a1 = rowb + (uint32_t)((((ch + 1) % 8) ^ (r & 7)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a0), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a1), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7]) : "memory");
      }
      // S buffer free for the tile after next; P visible to the tensor core
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_s_empty + 8 * buf) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_p_full) : "memory");
      l = l * corr + ls;
      m = m_new;
      // fold O_t = P V into the running output
      ok = mbar_wait(b_o_full, (uint32_t)j & 1u, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(lane_base + O_COL + (uint32_t)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i) o[c0 + i] = o[c0 + i] * corr + __uint_as_float(v[i]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_o_empty) : "memory");
    }
    if (ok && qi < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (b * p.S + qi) * (int64_t)p.nh * D + (int64_t)h * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 pr = __floats2bfloat162_rn(o[c0 + 2 * i] * inv, o[c0 + 2 * i + 1] * inv);
          w[i] = *(const uint32_t*)&pr;
        }
        *(uint4*)(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(NCOLS) : "memory");
  }
}

template <int D, int FA_BK>
int launch_fa(cg_ctx* c, const AttnArgs& a) {
  constexpr size_t smem =
      (size_t)(D / 64) * (128 + 4 * FA_BK) * 128 + (size_t)(FA_BK / 64) * 128 * 128 + (FA_BK == 64 ? 0 : 1024) + 160;
  static bool configured = false;
  if (!configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_attn_fa<D, FA_BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  CG_TRY(make_map(c, &mq, a.q, a.B * a.S, (int64_t)a.nh * D, (int64_t)a.nh * D, 128));
  CG_TRY(make_map(c, &mk, a.k_cache, a.B * a.nkv * a.Tmax, D, D, FA_BK));
  CG_TRY(make_map(c, &mv, a.v_cache, a.B * a.nkv * a.Tmax, D, D, FA_BK));
  FaArgs p;
  p.out = a.out;
  p.S = a.S; p.pos0 = a.pos0; p.Tmax = a.Tmax;
  p.nh = a.nh; p.nkv = a.nkv;
  p.scale_log2e = 1.4426950408889634f / sqrtf((float)D);
  p.err = c->core->dev_err;
  dim3 grid((unsigned)((a.S + FA_BQ - 1) / FA_BQ), (unsigned)a.nh, (unsigned)a.B);
  CG_CUDA(c, launch_kernel(c, k_attn_fa<D, FA_BK>, grid, dim3(192), smem, 1, mq, mk, mv, p));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace

bool attn_fa_supported(const AttnArgs& a) {
  return (a.d == 64 || a.d == 128) && a.window <= 0 && a.softcap <= 0.f && !a.pos_dev && a.S >= 64 &&
         a.B * a.S < 2147483647ll && a.B * a.nkv * a.Tmax < 2147483647ll && ((uintptr_t)a.q % 16) == 0 &&
         ((uintptr_t)a.k_cache % 16) == 0 && ((uintptr_t)a.v_cache % 16) == 0;
}

int k_launch_attn_fa(cg_ctx* c, const AttnArgs& a) {
  if (a.B == 0 || a.S == 0) return CG_OK;
  const bool k64 = c->opt_fa == 2;  // 64-key tiles: two CTAs per SM
  if (a.d == 64) return k64 ? launch_fa<64, 64>(c, a) : launch_fa<64, 128>(c, a);
  return k64 ? launch_fa<128, 64>(c, a) : launch_fa<128, 128>(c, a);
}

}  // namespace cg
