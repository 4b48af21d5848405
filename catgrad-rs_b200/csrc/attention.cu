// attention.cu — fused attention over the device KV cache.
//
// What the reference computes with materialised [1, nh, S, S] scores
// (catgrad-llm/src/models/llama.rs:97-108: q k^T / sqrt(d) + causal mask -> softmax -> v,
// after repeat_kv, catgrad-llm/src/helpers.rs:147-161) is done here without the S x S
// matrix: an online-softmax pass over key tiles.  Query head h reads kv head h / rep, the
// order repeat_kv produces.  Masked scores are dropped, which equals adding f32::MIN before
// the softmax (exp underflows to 0).
//
// BQ-query x 64-key tiles (BQ = 128 with 8 warps for head sizes up to 128, 64 with 4 warps
// for 256), bf16 mma.sync with f32 accumulation.  Key/value tiles arrive by cp.async into two
// shared-memory buffers, so the loads of tile i+1 overlap the math of tile i; query tiles are
// scheduled longest first (under the causal mask the last tile of a row has the most keys).
// (The one-token decode step has its own fused kernel.)
#include "kernels.h"
#include "mma.cuh"

#include <algorithm>

namespace cg {

namespace {

__device__ __forceinline__ float tanh_sig(float x) { return 2.f / (1.f + __expf(-2.f * x)) - 1.f; }

// ------------------------------------------------------------------ prefill ----------
template <int D, int BQ, int NBUF>
__global__ void __launch_bounds__(BQ * 2, D <= 64 ? 2 : 1) k_attn_prefill(AttnArgs a, float scale) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int BKV = 64, LD = D + 8, NT = BQ * 2;  // padded rows: conflict-free ldmatrix
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* sq = (__nv_bfloat16*)smem;
  __nv_bfloat16* sk = sq + BQ * LD;          // [NBUF][BKV][LD]
  __nv_bfloat16* sv = sk + NBUF * BKV * LD;  // [NBUF][BKV][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int kvh = h / (a.nh / a.nkv);
  const int64_t q0 = (int64_t)qt * BQ;
  const __nv_bfloat16* qbase = a.q + (b * a.S) * (int64_t)a.nh * D + (int64_t)h * D;
  const __nv_bfloat16* kbase = a.k_cache + ((b * a.nkv + kvh) * a.Tmax) * (int64_t)D;
  const __nv_bfloat16* vbase = a.v_cache + ((b * a.nkv + kvh) * a.Tmax) * (int64_t)D;

  // Q tile -> shared (rows past S are zero)
  constexpr int CH = D / 8;  // 16-byte chunks per row
  for (int i = tid; i < BQ * CH; i += NT) {
    const int r = i / CH, ch = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (q0 + r < a.S) v = *(const uint4*)(qbase + (q0 + r) * (int64_t)a.nh * D + ch * 8);
    *(uint4*)(sq + r * LD + ch * 8) = v;
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  const int r_in = lane >> 2, cq = (lane & 3) * 2;
  const int64_t qpos[2] = {a.pos0 + q0 + warp * 16 + r_in, a.pos0 + q0 + warp * 16 + r_in + 8};
  const int64_t kv_len = a.pos0 + a.S;
  const int64_t last_q = a.pos0 + std::min<int64_t>(a.S, q0 + BQ) - 1;  // last query position of this tile
  int64_t first_k = 0;
  if (a.window > 0) first_k = std::max<int64_t>(0, a.pos0 + q0 - a.window + 1);
  const int64_t kt0 = first_k / BKV, kt1 = last_q / BKV;  // inclusive key tile range

  const uint32_t sq_u = (uint32_t)__cvta_generic_to_shared(sq);
  const uint32_t sk_u = (uint32_t)__cvta_generic_to_shared(sk);
  const uint32_t sv_u = (uint32_t)__cvta_generic_to_shared(sv);
  const float LOG2E = 1.4426950408889634f;

  // asynchronous copy of key/value tile kt into buffer buf (rows past the context are zero)
  auto load_kv = [&](int buf, int64_t kt) {
    const int64_t k0 = kt * BKV;
    for (int i = tid; i < BKV * CH; i += NT) {
      const int r = i / CH, ch = i - r * CH;
      const bool in = k0 + r < kv_len;
      const int64_t off = in ? (k0 + r) * (int64_t)D + ch * 8 : 0;
      const uint32_t d = (uint32_t)(((buf * BKV + r) * LD + ch * 8) * 2);
      cp_async16(sk_u + d, kbase + off, in ? 16 : 0);
      cp_async16(sv_u + d, vbase + off, in ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (kt0 <= kt1) load_kv(0, kt0);

  for (int64_t kt = kt0; kt <= kt1; ++kt) {
    const int64_t k0 = kt * BKV;
    const int buf = NBUF == 2 ? (int)((kt - kt0) & 1) : 0;
    if (NBUF == 2 && kt < kt1) {
      load_kv(buf ^ 1, kt + 1);  // that buffer was last read two tiles ago, before the barrier that ended the previous tile
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();  // tile kt (and, the first time, Q) visible to every warp
    const uint32_t sk_b = sk_u + (uint32_t)(buf * BKV * LD * 2), sv_b = sv_u + (uint32_t)(buf * BKV * LD * 2);

    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[BKV / 8][4];
#pragma unroll
    for (int j = 0; j < BKV / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      {
        const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int col = kk * 16 + 8 * (lane >> 4);
        ldsm_x4(sq_u + (row * LD + col) * 2, a0, a1, a2, a3);
      }
#pragma unroll
      for (int j = 0; j < BKV / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = j * 8 + (lane & 7) + 8 * (lane >> 4);
        const int col = kk * 16 + 8 * ((lane >> 3) & 1);
        ldsm_x4(sk_b + (key * LD + col) * 2, b0, b1, b2, b3);
        mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    // scale, soft-cap, mask; row maxima
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < BKV / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t kpos = k0 + j * 8 + cq + (e & 1);
        const int64_t qp = qpos[e >> 1];
        float v = s[j][e] * scale;
        if (a.softcap > 0.f) v = a.softcap * tanh_sig(v / a.softcap);
        const bool keep = kpos <= qp && kpos < kv_len && (a.window <= 0 || kpos > qp - a.window);
        v = keep ? v : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(mrow[r], mx[r]);
      msafe[r] = mnew == -INFINITY ? 0.f : mnew;
      corr[r] = exp2f((mrow[r] - msafe[r]) * LOG2E);  // 0 when mrow is -inf
      mrow[r] = mnew;
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < BKV / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f((s[j][e] - msafe[e >> 1]) * LOG2E);
        s[j][e] = p;
        ls[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      ls[r] += __shfl_xor_sync(0xffffffffu, ls[r], 1);
      ls[r] += __shfl_xor_sync(0xffffffffu, ls[r], 2);
      lrow[r] = lrow[r] * corr[r] + ls[r];
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int col = j * 8 + 8 * (lane >> 4);
        ldsm_x4_t(sv_b + (key * LD + col) * 2, b0, b1, b2, b3);
        mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // every warp is done with this buffer before a later copy overwrites it
    if (NBUF == 1 && kt < kt1) load_kv(0, kt + 1);
  }

  // normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int64_t qi = q0 + warp * 16 + r_in + 8 * r;
    if (qi >= a.S) continue;
    const float inv = lrow[r] > 0.f ? 1.f / lrow[r] : 0.f;
    __nv_bfloat16* dst = a.out + (b * a.S + qi) * (int64_t)a.nh * D + (int64_t)h * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
      *(__nv_bfloat162*)(dst + j * 8 + cq) = v;
    }
  }
}

template <int D, int BQ, int NBUF>
int launch_prefill(cg_ctx* c, const AttnArgs& a) {
  constexpr size_t smem = (size_t)(BQ + 2 * NBUF * 64) * (D + 8) * 2;
  static PerDeviceFlag configured_on;
  bool& configured = configured_on.at(c->core->device);
  if (!configured && smem > 48 * 1024) {
    CG_CUDA(c, cudaFuncSetAttribute(k_attn_prefill<D, BQ, NBUF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid((unsigned)((a.S + BQ - 1) / BQ), (unsigned)a.nh, (unsigned)a.B);
  const float scale = 1.0f / sqrtf((float)D);
  CG_CUDA(c, launch_kernel(c, k_attn_prefill<D, BQ, NBUF>, grid, dim3(BQ * 2), smem, 1, a, scale));
  CG_LAUNCHED(c);
  return CG_OK;
}

int check(cg_ctx* c, const AttnArgs& a) {
  if (a.nkv <= 0 || a.nh % a.nkv) return fail(c, CG_ERR_SHAPE, "attention: heads must be a multiple of kv heads");
  if (a.d != 64 && a.d != 128 && a.d != 256) return fail(c, CG_ERR_UNSUPPORTED, "attention: head_dim must be 64, 128 or 256");
  if (a.pos0 + a.S > a.Tmax) return fail(c, CG_ERR_SHAPE, "attention: KV cache capacity exceeded");
  if (a.B > 65535 || a.nh > 65535) return fail(c, CG_ERR_UNSUPPORTED, "attention: too many rows or heads");
  return CG_OK;
}

}  // namespace

int k_launch_attn_prefill(cg_ctx* c, const AttnArgs& a) {
  CG_TRY(check(c, a));
  if (a.B == 0 || a.S == 0) return CG_OK;
  if (c->opt_fa && attn_fa_supported(a)) return k_launch_attn_fa(c, a);
  switch (a.d) {
    case 64: return launch_prefill<64, 128, 2>(c, a);
    case 128: return launch_prefill<128, 128, 2>(c, a);
    default: return launch_prefill<256, 64, 1>(c, a);
  }
}

}  // namespace cg

using namespace cg;

extern "C" int32_t cg_fused_attention(cg_ctx* c, const cg_tensor* q, const cg_tensor* k, const cg_tensor* v, int64_t window,
                                      float softcap, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !q || !k || !v || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (q->tag != CG_F32 || k->tag != CG_F32 || v->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "attention wants F32 tensors");
  if (q->rank != 4 || k->rank != 4 || v->rank != 4) return fail(c, CG_ERR_SHAPE, "attention wants [b, heads, s, d]");
  const int64_t B = q->dims[0], nh = q->dims[1], S = q->dims[2], d = q->dims[3], nkv = k->dims[1];
  for (int i = 0; i < 4; ++i)
    if (k->dims[i] != v->dims[i]) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  if (k->dims[0] != B || k->dims[2] != S || k->dims[3] != d) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  // bf16 copies in the layouts the kernel reads: q [B*S, nh*d], k/v [B, nkv, S, d]
  Hold qt, qb, kb, vb, ob, r;
  {
    cg_tensor* t = nullptr;
    CG_TRY(cg_transpose(c, q, 1, 2, &t));  // [B, S, nh, d] view
    qt.t = t;
  }
  CG_TRY(cg_to_bf16(c, qt.t, &qb.t));
  CG_TRY(cg_to_bf16(c, k, &kb.t));
  CG_TRY(cg_to_bf16(c, v, &vb.t));
  int64_t od[4] = {B, S, nh, d};
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, od, 4, &ob.t));
  AttnArgs a;
  a.q = (const __nv_bfloat16*)qb.t->data();
  a.k_cache = (const __nv_bfloat16*)kb.t->data();
  a.v_cache = (const __nv_bfloat16*)vb.t->data();
  a.out = (__nv_bfloat16*)ob.t->data();
  a.B = B; a.S = S; a.pos0 = 0; a.Tmax = S; a.pos_dev = nullptr;
  a.nh = (int)nh; a.nkv = (int)nkv; a.d = (int)d;
  a.window = window; a.softcap = softcap; a.scratch = nullptr;
  CG_TRY(k_launch_attn_prefill(c, a));
  // back to [B, nh, S, d] f32
  Hold ot;
  {
    cg_tensor* t = nullptr;
    CG_TRY(cg_transpose(c, ob.t, 1, 2, &t));
    ot.t = t;
  }
  CG_TRY(cg_to_f32(c, ot.t, &r.t));
  *out = r.take();
  return CG_OK;
}
