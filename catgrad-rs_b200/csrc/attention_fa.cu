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

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
      const int k0 = j * FA_BK;
      // a key column c of this tile is visible to this row iff c <= lim (causal mask)
      const int64_t lim64 = qpos - k0;
      const int lim = lim64 > FA_BK ? FA_BK : (lim64 < -1 ? -1 : (int)lim64);
      const bool diag = (int64_t)k0 + FA_BK - 1 > p.pos0 + q0;  // uniform: some key may be masked for some row
      const uint32_t s_addr = lane_base + buf * S_COLS;
      constexpr int NCH = FA_BK / 32;
      uint32_t va[32], vb[32];
      // pass 1: row maximum of the visible scores.  The loads are double-buffered: chunk c+1 is
      // in flight while chunk c is reduced.
      float mx = -INFINITY;
      tmem_ld32(s_addr, va);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t* cur = (c & 1) ? vb : va;
        uint32_t* nxt = (c & 1) ? va : vb;
        if (c + 1 < NCH) tmem_ld32(s_addr + (uint32_t)(c + 1) * 32u, nxt);
        if (!diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(cur[i]));
        } else {
          const int rel = lim - c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = i <= rel ? fmaxf(mx, __uint_as_float(cur[i])) : mx;
        }
        if (c + 1 < NCH) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      const float m_new = fmaxf(m, mx);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float corr = fast_exp2((m - m_safe) * p.scale_log2e);  // 0 while m is -inf
      const float mc = m_safe * p.scale_log2e;
      // the previous tile's P must have been consumed before it is overwritten
      if (j >= 1) {
        ok = mbar_wait(b_p_empty, ((uint32_t)j & 1u) ^ 1u, cta_abort, p.err);
        if (!ok) break;
      }
      // pass 2: p = exp2(s * scale * log2 e - m * scale * log2 e), row sum, bf16 P into the swizzled tile
      float ls = 0.f;
      tmem_ld32(s_addr, va);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t* cur = (c & 1) ? vb : va;
        uint32_t* nxt = (c & 1) ? va : vb;
        if (c + 1 < NCH) tmem_ld32(s_addr + (uint32_t)(c + 1) * 32u, nxt);
        const int rel = lim - c * 32;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = fast_exp2(fmaf(__uint_as_float(cur[i]), p.scale_log2e, -mc));
          float e1 = fast_exp2(fmaf(__uint_as_float(cur[i + 1]), p.scale_log2e, -mc));
          if (diag) {
            e0 = i <= rel ? e0 : 0.f;
            e1 = i + 1 <= rel ? e1 : 0.f;
          }
          ls += e0 + e1;
          const __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
          pk[i / 2] = *(const uint32_t*)&pr;
        }
        // four 16-byte chunks of row r: chunk index ch = 4 c + t; sub-tile ch / 8, position (ch % 8) ^ (r % 8)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int ch = 4 * c + t;
          const uint32_t a = sp + (uint32_t)(ch / 8) * BOX + (uint32_t)r * 128u + (uint32_t)(((ch % 8) ^ (r & 7)) * 16);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pk[4 * t]), "r"(pk[4 * t + 1]), "r"(pk[4 * t + 2]),
                       "r"(pk[4 * t + 3])
                       : "memory");
        }
        if (c + 1 < NCH) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      // S buffer free for the tile after next; P visible to the tensor core
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_s_empty + 8 * buf) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_p_full) : "memory");
      l = l * corr + ls;
      m = m_new;
      // fold O_t = P V into the running output (same double-buffered loads)
      ok = mbar_wait(b_o_full, (uint32_t)j & 1u, cta_abort, p.err);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      tmem_ld32(lane_base + O_COL, va);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t* cur = (c & 1) ? vb : va;
        uint32_t* nxt = (c & 1) ? va : vb;
        if (c + 1 < D / 32) tmem_ld32(lane_base + O_COL + (uint32_t)(c + 1) * 32u, nxt);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], corr, __uint_as_float(cur[i]));
        if (c + 1 < D / 32) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
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
