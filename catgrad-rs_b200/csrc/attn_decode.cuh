// attn_decode.cuh — the attention block of a decode step for one (row, kv head, context slice),
// as a device function shared by the stand-alone kernel (attn_decode.cu: one CTA per item, the
// slices of a pair forming a thread-block cluster) and the resident decode kernel
// (decode_resident.cu: 128 threads of a resident CTA work through a list of items).
//
// The caller supplies an environment:
//   tid()            0..127, the thread's index among the 128 threads that run the item
//   sync_cta()       barrier among those 128 threads
//   sync_group()     barrier among the CTAs that hold the slices of one (row, kv head),
//                    including a barrier among each CTA's own 128 threads
//   cluster_rank(s)  cluster rank of the CTA that holds slice s
//   kPush / landing()  kPush: the slices' partial results are PUSHED into a landing area (of
//                    attn_dec_landing_bytes(), shared memory that nothing else uses) of the CTA that
//                    finishes them, so one group barrier suffices and nobody waits before leaving;
//                    otherwise the finishing CTA reads the partials where they lie (two barriers)
//   settle(pos)      called once the first K/V tiles have been requested with a position that may
//                    be one step old: waits for whatever the caller's inputs depend on and returns
//                    the position to use (cached keys never change, so an early request is either
//                    right or is repeated)
#pragma once

#include "kernels.h"
#include "mma.cuh"

namespace cg {

constexpr int ATTN_MAX_REP = 8;  // query heads per kv head: rows 0..7 of the 16-row MMA tile

__device__ __forceinline__ float attn_tanh_sig(float x) { return 2.f / (1.f + __expf(-2.f * x)) - 1.f; }
__device__ __forceinline__ float attn_ld_dsmem(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// shared memory one item needs
template <int D>
__host__ __device__ constexpr size_t attn_dec_smem_bytes() {
  return (size_t)(16 * (D + 8) + 8 * (D > 128 ? 16 : 32) * (D + 8)) * 2 + (size_t)(2 * D + 8 * ATTN_MAX_REP + 16) * 4;
}

// landing area of the push form: {max, sum} per source slice and head, then per source slice the
// output values the CTA finishes (at most 8 slices; up to rep * D / 128 + 8 blocks of 128 values)
__host__ __device__ constexpr size_t attn_dec_landing_bytes() { return (size_t)(8 * ATTN_MAX_REP * 2 + (16 + 8) * 128) * 4; }

// KT = keys per warp tile: 32, or 16 for head size 256 so that a CTA's tiles fit a third of an
// SM's shared memory.
template <int D, class Env>
__device__ __forceinline__ void attn_dec_item(const AttnDecArgs& a, float scale, int kvh, int64_t b, int split, int64_t pos_early,
                                              uint8_t* smem, Env& env) {
  constexpr int KT = D > 128 ? 16 : 32;
  constexpr int MAX_REP = ATTN_MAX_REP;
  constexpr int LD = D + 8;     // padded rows: conflict-free ldmatrix
  constexpr int CH = D / 8;     // 16-byte chunks per row
  constexpr int NT = D / 8;     // output n-tiles
  __nv_bfloat16* qt = (__nv_bfloat16*)smem;              // [16][LD] query heads (rows >= rep are zero)
  __nv_bfloat16* kt = qt + 16 * LD;                      // [4 warps][KT][LD] key tiles
  __nv_bfloat16* vt = kt + 4 * KT * LD;                  // [4 warps][KT][LD] value tiles
  float* fl = (float*)(vt + 4 * KT * LD);
  float* knew = fl;                                      // [D] the new key (bf16-rounded)
  float* vnew = knew + D;                                // [D]
  float* red_m = vnew + D;                               // [4][MAX_REP]
  float* red_l = red_m + 4 * MAX_REP;                    // [4][MAX_REP]
  float* hsq = red_l + 4 * MAX_REP;                      // [MAX_REP + 1] per-head rms (norm), padded to 16
  float* red_o = (float*)kt;                             // [4][MAX_REP][D] f32, reuses the tiles after the loop

  const int tid = env.tid(), warp = tid >> 5, lane = tid & 31;
  const int rep = a.nh / a.nkv;
  const int half = D / 2;
  // pos: position of the new token = number of cached keys.  The projected row is read with
  // L2 loads: in the resident kernel another CTA wrote it earlier in the same launch.
  __nv_bfloat16* kbase = a.k_cache + ((b * a.nkv + kvh) * a.Tmax) * (int64_t)D;
  __nv_bfloat16* vbase = a.v_cache + ((b * a.nkv + kvh) * a.Tmax) * (int64_t)D;

  // this CTA's slice of the cached keys [lo, pos)
  int64_t pos = pos_early, t0 = 0, t1 = 0;
  auto plan = [&]() {
    int64_t lo = 0;
    if (a.window > 0) lo = max((int64_t)0, pos - a.window + 1);
    const int64_t span = pos - lo;
    int64_t per = (span + a.splits - 1) / a.splits;
    per = (per + KT - 1) / KT * KT;
    t0 = lo + split * per;
    t1 = min(pos, t0 + per);
  };
  plan();

  __nv_bfloat16* kw = kt + (size_t)warp * KT * LD;
  __nv_bfloat16* vw = vt + (size_t)warp * KT * LD;
  const uint32_t kw_u = (uint32_t)__cvta_generic_to_shared(kw);
  const uint32_t vw_u = (uint32_t)__cvta_generic_to_shared(vw);
  const uint32_t qt_u = (uint32_t)__cvta_generic_to_shared(qt);

  // request the first chunk of this warp now: it does not depend on q
  auto request = [&](int64_t c0) {
    // KT rows x CH chunks, 8 (or more) lanes per row: fully coalesced 16-byte copies
    for (int i = lane; i < KT * CH; i += 32) {
      const int r = i / CH, ch = i - r * CH;
      const int64_t key = c0 + r;
      const bool ok = key < t1;
      const int64_t kc = ok ? key : t0;
      cp_async16(kw_u + (uint32_t)(r * LD + ch * 8) * 2u, kbase + kc * (int64_t)D + ch * 8, ok ? 16 : 0);
      cp_async16(vw_u + (uint32_t)(r * LD + ch * 8) * 2u, vbase + kc * (int64_t)D + ch * 8, ok ? 16 : 0);
    }
  };
  int64_t c0 = t0 + warp * KT;
  if (c0 < t1) request(c0);
  {
    const int64_t pos_now = env.settle(pos);
    if (pos_now != pos) {  // the early position was stale: let the copies land, then ask again
      cp_async_wait_all();
      __syncwarp();
      pos = pos_now;
      plan();
      c0 = t0 + warp * KT;
      if (c0 < t1) request(c0);
    }
  }

  // ---- 1. q, k, v of the new token ----
  const int heads = a.nh + 2 * a.nkv;
  const float* row = a.qkv + b * (int64_t)heads * D;
  const float* qsrc = row + (int64_t)kvh * rep * D;
  const float* ksrc = row + ((int64_t)a.nh + kvh) * D;
  const float* vsrc = row + ((int64_t)a.nh + a.nkv + kvh) * D;
  if (a.q_gamma) {
    // per-head RMSNorm over d for the rep query heads and the key head
    for (int h = warp; h <= rep; h += 4) {
      const float* src = h < rep ? qsrc + h * D : ksrc;
      float ss = 0.f;
      for (int e = lane; e < D; e += 32) { const float v = __ldcg(src + e); ss += v * v; }
#pragma unroll
      for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) hsq[h] = sqrtf(ss / (float)D + a.norm_eps);
    }
    env.sync_cta();
  }
  for (int i = tid; i < 16 * half; i += 128) {
    const int h = i / half, j = i - h * half;
    if (h < rep) {
      float x1 = __ldcg(qsrc + h * D + j), x2 = __ldcg(qsrc + h * D + j + half);
      if (a.q_gamma) {
        const float g1 = a.norm_plus_one ? 1.f + a.q_gamma[j] : a.q_gamma[j];
        const float g2 = a.norm_plus_one ? 1.f + a.q_gamma[j + half] : a.q_gamma[j + half];
        x1 = x1 / hsq[h] * g1;
        x2 = x2 / hsq[h] * g2;
      }
      const float cs = a.cos_t[pos * half + j], sn = a.sin_t[pos * half + j];
      qt[h * LD + j] = __float2bfloat16_rn(cs * x1 - sn * x2);
      qt[h * LD + j + half] = __float2bfloat16_rn(cs * x2 + sn * x1);
    } else {
      qt[h * LD + j] = __float2bfloat16_rn(0.f);
      qt[h * LD + j + half] = __float2bfloat16_rn(0.f);
    }
  }
  for (int j = tid; j < half; j += 128) {
    float x1 = __ldcg(ksrc + j), x2 = __ldcg(ksrc + j + half);
    if (a.q_gamma) {
      const float g1 = a.norm_plus_one ? 1.f + a.k_gamma[j] : a.k_gamma[j];
      const float g2 = a.norm_plus_one ? 1.f + a.k_gamma[j + half] : a.k_gamma[j + half];
      x1 = x1 / hsq[rep] * g1;
      x2 = x2 / hsq[rep] * g2;
    }
    const float cs = a.cos_t[pos * half + j], sn = a.sin_t[pos * half + j];
    const __nv_bfloat16 k1 = __float2bfloat16_rn(cs * x1 - sn * x2), k2 = __float2bfloat16_rn(cs * x2 + sn * x1);
    const __nv_bfloat16 v1 = __float2bfloat16_rn(__ldcg(vsrc + j)), v2 = __float2bfloat16_rn(__ldcg(vsrc + j + half));
    knew[j] = __bfloat162float(k1);
    knew[j + half] = __bfloat162float(k2);
    vnew[j] = __bfloat162float(v1);
    vnew[j + half] = __bfloat162float(v2);
    if (split == 0) {  // append to the cache for the following steps
      kbase[pos * D + j] = k1;
      kbase[pos * D + j + half] = k2;
      vbase[pos * D + j] = v1;
      vbase[pos * D + j + half] = v2;
    }
  }
  env.sync_cta();

  // ---- 2. this warp's chunks of 32 keys: S = Q K^T, online softmax, O += P V ----
  // A thread owns head r = lane / 4 (rows 8..15 of the MMA tile are padding) and, per 8-key
  // or 8-column tile, the two columns 2 * (lane % 4) + {0, 1}.
  const int hr = lane >> 2, cq = (lane & 3) * 2;
  float m = -INFINITY, l = 0.f;
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  // slice 0, warp 0 also owns the new token: one more chunk whose only live key is row 0
  const bool owns_new = split == 0 && warp == 0;
  bool do_new = false;
  while (true) {
    int64_t limit;  // live keys of this chunk are [c0, limit)
    if (c0 < t1) {
      limit = t1;
      cp_async_wait_all();
      __syncwarp();
    } else if (owns_new && !do_new) {
      do_new = true;
      // build the one-row chunk in the tiles
      for (int e = lane; e < D; e += 32) {
        kw[e] = __float2bfloat16_rn(knew[e]);
        vw[e] = __float2bfloat16_rn(vnew[e]);
      }
      for (int i = lane; i < (KT - 1) * CH; i += 32) {
        const int r = 1 + i / CH, ch = i % CH;
        *(uint4*)(vw + r * LD + ch * 8) = make_uint4(0u, 0u, 0u, 0u);  // p = 0 times NaN garbage must not happen
        *(uint4*)(kw + r * LD + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
      limit = 1;  // in units relative to a chunk start of 0
    } else {
      break;
    }
    const int64_t cbase = do_new ? 0 : c0;

    float s[KT / 8][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      {
        const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
        const int col = kk * 16 + 8 * (lane >> 4);
        ldsm_x4(qt_u + (uint32_t)(r * LD + col) * 2u, a0, a1, a2, a3);
      }
#pragma unroll
      for (int j = 0; j < KT / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = j * 8 + (lane & 7) + 8 * (lane >> 4);
        const int col = kk * 16 + 8 * ((lane >> 3) & 1);
        ldsm_x4(kw_u + (uint32_t)(key * LD + col) * 2u, b0, b1, b2, b3);
        mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // scale, soft-cap, mask; this head's maximum over the chunk
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float v = s[j][e] * scale;
        if (a.softcap > 0.f) v = a.softcap * attn_tanh_sig(v / a.softcap);
        const bool keep = cbase + j * 8 + cq + e < limit;
        v = keep ? v : -INFINITY;
        s[j][e] = v;
        mx = fmaxf(mx, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mnew = fmaxf(m, mx);  // finite: the first key of every chunk is live
    const float corr = __expf(m - mnew);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p = __expf(s[j][e] - mnew);
        s[j][e] = p;
        sum += p;
      }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l = l * corr + sum;
    m = mnew;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= corr;
      o[j][1] *= corr;
    }
    // O += P V; rows 8..15 of P are zero
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int col = j * 8 + 8 * (lane >> 4);
        ldsm_x4_t(vw_u + (uint32_t)(key * LD + col) * 2u, b0, b1, b2, b3);
        mma_bf16(o[j], a0, 0u, a2, 0u, b0, b1);
        mma_bf16(o[j + 1], a0, 0u, a2, 0u, b2, b3);
      }
    }
    __syncwarp();
    if (do_new) break;
    c0 += 4 * KT;
    if (c0 < t1) request(c0);
  }

  // ---- 3. merge the four warps in this CTA, then the slices across the cluster ----
  env.sync_cta();  // all tiles are dead: reuse their space
  if (hr < rep) {
    if ((lane & 3) == 0) { red_m[warp * MAX_REP + hr] = m; red_l[warp * MAX_REP + hr] = l; }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      red_o[(warp * MAX_REP + hr) * D + j * 8 + cq] = o[j][0];
      red_o[(warp * MAX_REP + hr) * D + j * 8 + cq + 1] = o[j][1];
    }
  }
  env.sync_cta();
  // this slice's partial: part[r] = {max, sum}, part_o[r][e], left in shared memory for the cluster
  float* part_ml = (float*)vt;                 // [MAX_REP][2]
  float* part_o = part_ml + 2 * MAX_REP;       // [MAX_REP][D]
  const int S = a.splits;
  const bool push = Env::kPush && a.push_merge && S > 1;
  // push form: output i is finished by slice (i / 128) % S, as its block number (i / 128) / S
  const int kmax = (rep * D + 128 * S - 1) / (128 * S);
  float* land_ml = nullptr;   // [8][MAX_REP][2]
  float* land_o = nullptr;    // [S][kmax][128]
  uint32_t land_u = 0;
  if (push) {
    land_ml = env.landing();
    land_o = land_ml + 8 * MAX_REP * 2;
    land_u = (uint32_t)__cvta_generic_to_shared(land_ml);
  }
  auto st_remote = [&](uint32_t local_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
  };
  for (int i = tid; i < rep * D; i += 128) {
    const int r = i / D, e = i - r * D;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_m[w * MAX_REP + r]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * MAX_REP + r];
      const float f = mw == -INFINITY ? 0.f : __expf(mw - mm);
      ll += red_l[w * MAX_REP + r] * f;
      oo += red_o[(w * MAX_REP + r) * D + e] * f;
    }
    if (push) {
      const int blk = i >> 7;
      st_remote(land_u + (uint32_t)(8 * MAX_REP * 2 + ((split * kmax + blk / S) << 7) + (i & 127)) * 4u, env.cluster_rank(blk % S), oo);
      if (e == 0)
        for (int s = 0; s < S; ++s) {
          st_remote(land_u + (uint32_t)((split * MAX_REP + r) * 2) * 4u, env.cluster_rank(s), mm);
          st_remote(land_u + (uint32_t)((split * MAX_REP + r) * 2 + 1) * 4u, env.cluster_rank(s), ll);
        }
      continue;
    }
    if (e == 0) { part_ml[2 * r] = mm; part_ml[2 * r + 1] = ll; }
    part_o[r * D + e] = oo;
  }
  if (push) {
    // one barrier: every slice's pushes are visible after it and nobody touches another CTA's
    // shared memory again
    env.sync_group();
    int k = 0;
    for (int i = tid + 128 * split; i < rep * D; i += 128 * S, ++k) {
      const int r = i / D;
      float ms[8], ls[8], os[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const bool in = s < S;
        ms[s] = in ? land_ml[(s * MAX_REP + r) * 2] : -INFINITY;
        ls[s] = in ? land_ml[(s * MAX_REP + r) * 2 + 1] : 0.f;
        os[s] = in ? land_o[((s * kmax + k) << 7) + tid] : 0.f;
      }
      float mm = -INFINITY;
#pragma unroll
      for (int s = 0; s < 8; ++s) mm = fmaxf(mm, ms[s]);
      float ll = 0.f, oo = 0.f;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const float f = ms[s] == -INFINITY ? 0.f : __expf(ms[s] - mm);
        ll += ls[s] * f;
        oo += os[s] * f;
      }
      a.out[(b * a.nh + kvh * rep + r) * (int64_t)D + (i - r * D)] = __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
    }
    return;
  }
  if (S == 1) {
    env.sync_cta();
    for (int i = tid; i < rep * D; i += 128) {
      const int r = i / D, e = i - r * D;
      const float ll = part_ml[2 * r + 1];
      a.out[(b * a.nh + kvh * rep + r) * (int64_t)D + e] = __float2bfloat16_rn(ll > 0.f ? part_o[i] / ll : 0.f);
    }
    env.sync_cta();  // the partials are read: the next item of a resident CTA may reuse the space
    return;
  }
  // the slices of one (row, kv head) are one thread-block cluster: merge over distributed
  // shared memory, each CTA finishing an interleaved share of the outputs
  env.sync_group();
  const uint32_t ml_u = (uint32_t)__cvta_generic_to_shared(part_ml);
  const uint32_t po_u = (uint32_t)__cvta_generic_to_shared(part_o);
  for (int i = tid + 128 * split; i < rep * D; i += 128 * S) {
    const int r = i / D;
    // all remote loads first (their latencies overlap), then the arithmetic; S <= 8
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const bool in = s < S;
      ms[s] = in ? attn_ld_dsmem(ml_u + (uint32_t)(2 * r) * 4u, env.cluster_rank(s)) : -INFINITY;
      ls[s] = in ? attn_ld_dsmem(ml_u + (uint32_t)(2 * r + 1) * 4u, env.cluster_rank(s)) : 0.f;
      os[s] = in ? attn_ld_dsmem(po_u + (uint32_t)i * 4u, env.cluster_rank(s)) : 0.f;
    }
    float mm = -INFINITY;
#pragma unroll
    for (int s = 0; s < 8; ++s) mm = fmaxf(mm, ms[s]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const float f = ms[s] == -INFINITY ? 0.f : __expf(ms[s] - mm);
      ll += ls[s] * f;
      oo += os[s] * f;
    }
    a.out[(b * a.nh + kvh * rep + r) * (int64_t)D + (i - r * D)] = __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
  }
  // nobody leaves while a peer may still read its shared memory
  env.sync_group();
}

}  // namespace cg
