// fused.cu — memory-bound fused kernels: each does in one pass over HBM what the reference
// spreads over a chain of primitive backend calls with materialised intermediates
// (catgrad/src/stdlib/nn/mod.rs:117-171, catgrad-llm/src/helpers.rs:120-271).
// Rows are reduced with warp shuffles; loads are 128-bit where the row length allows.
#include "act.cuh"
#include "kernels.h"
#include "peer.cuh"

#include <algorithm>

namespace cg {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum / max (blockDim multiple of 32, <= 1024); sh holds 32 floats
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  v = lane < nw ? sh[lane] : 0.f;
  return warp_sum(v);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  v = lane < nw ? sh[lane] : -INFINITY;
  return warp_max(v);
}

__global__ void k_embed(const uint32_t* tokens, int64_t tok_ld, int64_t tok_off, int64_t S, const void* table, int st,
                        int64_t vocab, int64_t H, float scale, float* out, int32_t* err) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t m = blockIdx.x;
  const int64_t b = m / S, sp = m - b * S;
  uint32_t t = tokens[b * tok_ld + tok_off + sp];
  if (t >= vocab) { if (threadIdx.x == 0) *err = DEV_INDEX; t = 0; }
  if (st == ST_BF16 && H % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    // eight values per thread: one 128-bit load, two 128-bit stores
    const uint4* row = (const uint4*)((const __nv_bfloat16*)table + (int64_t)t * H);
    float4* o = (float4*)(out + m * H);
    for (int64_t i = threadIdx.x; i < H / 8; i += blockDim.x) {
      const uint4 r = row[i];
      const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&r.x), b2 = __bfloat1622float2(*(const __nv_bfloat162*)&r.y);
      const float2 c2 = __bfloat1622float2(*(const __nv_bfloat162*)&r.z), d2 = __bfloat1622float2(*(const __nv_bfloat162*)&r.w);
      o[2 * i] = make_float4(a.x * scale, a.y * scale, b2.x * scale, b2.y * scale);
      o[2 * i + 1] = make_float4(c2.x * scale, c2.y * scale, d2.x * scale, d2.y * scale);
    }
  } else if (st == ST_BF16) {
    const __nv_bfloat162* row = (const __nv_bfloat162*)((const __nv_bfloat16*)table + (int64_t)t * H);
    float2* o = (float2*)(out + m * H);
    for (int64_t i = threadIdx.x; i < H / 2; i += blockDim.x) {
      float2 v = __bfloat1622float2(row[i]);
      o[i] = make_float2(v.x * scale, v.y * scale);
    }
    if ((H & 1) && threadIdx.x == 0)
      out[m * H + H - 1] = __bfloat162float(((const __nv_bfloat16*)table)[(int64_t)t * H + H - 1]) * scale;
  } else {
    const float* row = (const float*)table + (int64_t)t * H;
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x) out[m * H + i] = row[i] * scale;
  }
}

// One block per row.  MODE 0: out f32, 1: out bf16, 2: x_acc += normed(y)
template <int MODE>
__global__ void k_rmsnorm(const float* x, int64_t ldx, const float* gamma, float eps, int plus_one, int64_t H, void* out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float sh[32];
  const int64_t m = blockIdx.x;
  const float* row = x + m * ldx;
  float ss = 0.f;
  const bool vec = (H % 4 == 0) && (ldx % 4 == 0) && (((uintptr_t)x & 15) == 0);
  if (vec && H <= (int64_t)blockDim.x * 16 && (((uintptr_t)gamma & 15) == 0) && (((uintptr_t)out & 15) == 0)) {
    // The row fits the block's registers (up to four 128-bit loads per thread, all issued before
    // the first use): one pass over HBM, no second read of the row.
    const float4* r4 = (const float4*)row;
    const int n4 = (int)(H / 4);
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = i < n4 ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    ss = block_sum(ss, sh);
    const float rms = sqrtf(ss / (float)H + eps);
    const float4* g4 = (const float4*)gamma;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i >= n4) break;
      float4 g = g4[i];
      if (plus_one) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
      const float4 r = make_float4(v[j].x / rms * g.x, v[j].y / rms * g.y, v[j].z / rms * g.z, v[j].w / rms * g.w);
      if (MODE == 0) {
        ((float4*)((float*)out + m * H))[i] = r;
      } else if (MODE == 1) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
        ((uint2*)((__nv_bfloat16*)out + m * H))[i] = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
      } else {
        float4* o = (float4*)((float*)out + m * H) + i;
        float4 a = *o;
        a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
        *o = a;
      }
    }
    return;
  }
  if (vec) {
    const float4* r4 = (const float4*)row;
    for (int64_t i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 v = r4[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x) ss += row[i] * row[i];
  }
  ss = block_sum(ss, sh);
  const float rms = sqrtf(ss / (float)H + eps);
  if (MODE == 1 && vec && (((uintptr_t)gamma & 15) == 0)) {
    // bf16 output: 128-bit loads (the row is hot in L1 / L2 after the first pass), 64-bit stores
    const float4* r4 = (const float4*)row;
    const float4* g4 = (const float4*)gamma;
    uint2* o2 = (uint2*)((__nv_bfloat16*)out + m * H);
    for (int64_t i = threadIdx.x; i < H / 4; i += blockDim.x) {
      const float4 v = r4[i];
      float4 g = g4[i];
      if (plus_one) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x / rms * g.x, v.y / rms * g.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z / rms * g.z, v.w / rms * g.w);
      o2[i] = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = plus_one ? 1.f + gamma[i] : gamma[i];
    const float v = row[i] / rms * g;
    if (MODE == 0) ((float*)out)[m * H + i] = v;
    else if (MODE == 1) ((__nv_bfloat16*)out)[m * H + i] = __float2bfloat16_rn(v);
    else ((float*)out)[m * H + i] += v;
  }
}

// Post-norm layers (catgrad-llm/src/models/gemma3.rs:192-238): x += rmsnorm(y; g1), and in the
// same pass the norm that the next block starts with, out = bf16(rmsnorm(x; g2)).  One block per row.
__global__ void k_rmsnorm_add_norm(const float* y, const float* g1, const float* g2, float eps, int plus_one, int64_t H, float* x,
                                   __nv_bfloat16* out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float sh[32];
  const int64_t m = blockIdx.x;
  const float* yr = y + m * H;
  float* xr = x + m * H;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) ss += yr[i] * yr[i];
  ss = block_sum(ss, sh);
  const float rms1 = sqrtf(ss / (float)H + eps);
  float s2 = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = plus_one ? 1.f + g1[i] : g1[i];
    const float v = xr[i] + yr[i] / rms1 * g;
    xr[i] = v;
    s2 += v * v;
  }
  s2 = block_sum(s2, sh);
  const float rms2 = sqrtf(s2 / (float)H + eps);
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = plus_one ? 1.f + g2[i] : g2[i];
    out[m * H + i] = __float2bfloat16_rn(xr[i] / rms2 * g);  // this thread's own store above
  }
}

// Tensor-parallel prefill: the row-parallel projections meet in a bf16 all-reduce; this adds the
// reduced rows to the f32 residual stream, x += t, and in the same pass writes the norm the next
// block starts with, out = bf16(rmsnorm(x; g)) (g null: the add only).  One block per row.
__global__ void k_add_bf16_norm(const __nv_bfloat16* t, const float* g, float eps, int plus_one, int64_t H, float* x,
                                __nv_bfloat16* out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float sh[32];
  const int64_t m = blockIdx.x;
  const __nv_bfloat162* tr = (const __nv_bfloat162*)(t + m * H);
  float2* xr = (float2*)(x + m * H);
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < H / 2; i += blockDim.x) {
    const float2 a = __bfloat1622float2(tr[i]);
    float2 v = xr[i];
    v.x += a.x;
    v.y += a.y;
    xr[i] = v;
    ss += v.x * v.x + v.y * v.y;
  }
  if (!g) return;
  ss = block_sum(ss, sh);
  const float rms = sqrtf(ss / (float)H + eps);
  __nv_bfloat162* o = (__nv_bfloat162*)(out + m * H);
  const float2* g2 = (const float2*)g;
  for (int64_t i = threadIdx.x; i < H / 2; i += blockDim.x) {
    const float2 v = xr[i];  // this thread's own store above
    float2 gg = g2[i];
    if (plus_one) { gg.x += 1.f; gg.y += 1.f; }
    o[i] = __floats2bfloat162_rn(v.x / rms * gg.x, v.y / rms * gg.y);
  }
}

__global__ void k_act_mul(const float* gu, int64_t F, int act, __nv_bfloat16* out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t m = blockIdx.y;
  const float* g = gu + m * 2 * F;
  const float* u = g + F;
  if ((F & 3) == 0) {
    // 128-bit loads, 64-bit stores
    const float4* g4 = (const float4*)g;
    const float4* u4 = (const float4*)u;
    uint2* o2 = (uint2*)(out + m * F);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < F / 4; i += (int64_t)gridDim.x * blockDim.x) {
      const float4 a = g4[i], b = u4[i];
      float r[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = act == 0 ? silu_f(r[j]) : gelu_f(r[j]);
      __nv_bfloat162 lo = __floats2bfloat162_rn(r[0] * b.x, r[1] * b.y), hi = __floats2bfloat162_rn(r[2] * b.z, r[3] * b.w);
      o2[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    }
    return;
  }
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < F; i += (int64_t)gridDim.x * blockDim.x) {
    const float a = act == 0 ? silu_f(g[i]) : gelu_f(g[i]);
    out[m * F + i] = __float2bfloat16_rn(a * u[i]);
  }
}
// 128-bit loads and stores, two independent vectors per thread and pass
__global__ void k_act_mul_f32_vec(const float4* g, const float4* u, int64_t n4, int act, float4* out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
    const int64_t k = i + stride;
    const float4 a0 = g[i], b0 = u[i];
    const bool two = k < n4;
    const float4 a1 = two ? g[k] : a0, b1 = two ? u[k] : b0;
    float4 r0, r1;
    r0.x = (act == 0 ? silu_f(a0.x) : gelu_f(a0.x)) * b0.x; r0.y = (act == 0 ? silu_f(a0.y) : gelu_f(a0.y)) * b0.y;
    r0.z = (act == 0 ? silu_f(a0.z) : gelu_f(a0.z)) * b0.z; r0.w = (act == 0 ? silu_f(a0.w) : gelu_f(a0.w)) * b0.w;
    r1.x = (act == 0 ? silu_f(a1.x) : gelu_f(a1.x)) * b1.x; r1.y = (act == 0 ? silu_f(a1.y) : gelu_f(a1.y)) * b1.y;
    r1.z = (act == 0 ? silu_f(a1.z) : gelu_f(a1.z)) * b1.z; r1.w = (act == 0 ? silu_f(a1.w) : gelu_f(a1.w)) * b1.w;
    out[i] = r0;
    if (two) out[k] = r1;
  }
}
__global__ void k_act_mul_f32(const float* g, const float* u, int64_t n, int act, float* out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float a = act == 0 ? silu_f(g[i]) : gelu_f(g[i]);
    out[i] = a * u[i];
  }
}

// one block per row: softmax(x) or softmax(cap * tanh(x / cap))
__global__ void k_softmax(const float* x, int64_t n, float softcap, float* out) {
  __shared__ float sh[32];
  const float* row = x + (int64_t)blockIdx.x * n;
  float* o = out + (int64_t)blockIdx.x * n;
  float mx = -3.4028234663852886e38f;  // the reference folds max from f32::MIN
  if ((n & 3) == 0 && n <= (int64_t)blockDim.x * 16 && (((uintptr_t)row & 15) == 0) && (((uintptr_t)o & 15) == 0)) {
    // register-resident row: one read and one write of HBM per element
    const float4* r4 = (const float4*)row;
    const int n4 = (int)(n / 4);
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      const float4 t = i < n4 ? r4[i] : make_float4(mx, mx, mx, mx);
      v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
    if (softcap > 0.f) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if ((int)threadIdx.x + (j >> 2) * (int)blockDim.x < n4) v[j] = softcap * tanh_f(v[j] / softcap);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) mx = fmaxf(mx, v[j]);
    mx = block_max(mx, sh);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const bool live = (int)threadIdx.x + (j >> 2) * (int)blockDim.x < n4;
      v[j] = live ? __expf(v[j] - mx) : 0.f;
      s += v[j];
    }
    s = block_sum(s, sh);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) ((float4*)o)[i] = make_float4(v[4 * j] / s, v[4 * j + 1] / s, v[4 * j + 2] / s, v[4 * j + 3] / s);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = row[i];
    if (softcap > 0.f) v = softcap * tanh_f(v / softcap);
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, sh);
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = row[i];
    if (softcap > 0.f) v = softcap * tanh_f(v / softcap);
    const float e = __expf(v - mx);
    o[i] = e;
    s += e;
  }
  s = block_sum(s, sh);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) o[i] = o[i] / s;
}

// cos/sin tables as rope_tables builds them (helpers.rs:164-193): f = i * (2/d) rounded
// twice, inv = 1 / theta^f, angle = pos * inv, all in f32; the transcendental functions go
// through double like the elementwise pow/sin/cos kernels do.
__global__ void k_rope_tables(float theta, int64_t T, int64_t half, float two_over_d, float* cos_t, float* sin_t) {
  const int64_t n = T * half;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t pos = i / half, j = i - pos * half;
    const float f = (float)j * two_over_d;
    const float freq = (float)pow((double)theta, (double)f);
    const float inv = 1.0f / freq;
    const float ang = (float)pos * inv;
    cos_t[i] = (float)cos((double)ang);
    sin_t[i] = (float)sin((double)ang);
  }
}

// Scaled variants (legacy/nn/rope.rs:32-201), every step in f32 and un-fused so that the table
// equals an f32 evaluation of the reference's expression tree operation by operation.
__global__ void k_rope_tables_scaled(float theta, RopeScaling rs, float yarn_low, float yarn_high, float mscale, int64_t T,
                                     int64_t half, float two_over_d, float* cos_t, float* sin_t) {
  const int64_t n = T * half;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t pos = i / half, j = i - pos * half;
    const float f = __fmul_rn((float)j, two_over_d);
    const float freq = (float)pow((double)theta, (double)f);
    float inv = __fdiv_rn(1.0f, freq);
    if (rs.kind == 1) {
      // rope.rs:49-93
      const float old_ctx = (float)rs.original_max_pos;
      const float low_wl = __fdiv_rn(old_ctx, rs.low_freq_factor), high_wl = __fdiv_rn(old_ctx, rs.high_freq_factor);
      const float wavelen = __fdiv_rn(6.2831855f, inv);  // 2 * PI in f32
      const bool low = wavelen > low_wl;
      const float inv1 = low ? __fdiv_rn(inv, rs.factor) : inv;
      const bool high = wavelen < high_wl;
      const float smooth = __fdiv_rn(__fsub_rn(__fdiv_rn(old_ctx, wavelen), rs.low_freq_factor),
                                     __fsub_rn(rs.high_freq_factor, rs.low_freq_factor));
      const float smoothed = __fadd_rn(__fmul_rn(smooth, inv1), __fdiv_rn(__fmul_rn(__fsub_rn(1.0f, smooth), inv1), rs.factor));
      inv = (!high && !low) ? smoothed : inv1;
    } else if (rs.kind == 2) {
      // rope.rs:139-185: ramp = clamp((j - low) / (high - low), 0, 1); extrapolation share = 1 - ramp
      float r = __fdiv_rn(__fsub_rn((float)j, yarn_low), __fsub_rn(yarn_high, yarn_low));
      r = fminf(fmaxf(r, 0.0f), 1.0f);
      const float ext = __fsub_rn(1.0f, r);
      const float interp = __fdiv_rn(inv, rs.factor);
      inv = __fadd_rn(__fmul_rn(interp, __fsub_rn(1.0f, ext)), __fmul_rn(inv, ext));
    }
    const float ang = __fmul_rn((float)pos, inv);
    float cs = (float)cos((double)ang), sn = (float)sin((double)ang);
    if (rs.kind == 2) { cs = __fmul_rn(cs, mscale); sn = __fmul_rn(sn, mscale); }
    cos_t[i] = cs;
    sin_t[i] = sn;
  }
}

// x [rows, S, d] -> cos * x + sin * rotate_half(x), position pos0 + s
__global__ void k_rope_apply(const float* x, const float* cos_t, const float* sin_t, int64_t S, int64_t d, int64_t pos0,
                             int64_t n, float* out) {
  const int64_t half = d / 2;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i % d, s = (i / d) % S;
    const int64_t j = e < half ? e : e - half;
    const float c = cos_t[(pos0 + s) * half + j], sn = sin_t[(pos0 + s) * half + j];
    const float rot = e < half ? -x[i + half] : x[i - half];
    out[i] = c * x[i] + sn * rot;
  }
}

// Four rotation pairs per thread: 128-bit loads of both halves of the head and of the tables,
// 128-bit stores.  x is [rows, S, d] with d / 2 a multiple of 4; n4 = rows * S * (d / 8) groups.
__global__ void k_rope_apply_vec(const float* x, const float* cos_t, const float* sin_t, int64_t S, int64_t d, int64_t pos0,
                                 int64_t n4, float* out) {
  const int64_t half = d / 2, per_row = half / 4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row, j = (i - r * per_row) * 4;   // r = row * S + s
    const int64_t s = r % S;
    const float4 x1 = *(const float4*)(x + r * d + j), x2 = *(const float4*)(x + r * d + half + j);
    const float4 c = *(const float4*)(cos_t + (pos0 + s) * half + j), sn = *(const float4*)(sin_t + (pos0 + s) * half + j);
    *(float4*)(out + r * d + j) = make_float4(c.x * x1.x + sn.x * -x2.x, c.y * x1.y + sn.y * -x2.y, c.z * x1.z + sn.z * -x2.z,
                                              c.w * x1.w + sn.w * -x2.w);
    *(float4*)(out + r * d + half + j) = make_float4(c.x * x2.x + sn.x * x1.x, c.y * x2.y + sn.y * x1.y, c.z * x2.z + sn.z * x1.z,
                                                     c.w * x2.w + sn.w * x1.w);
  }
}

// One warp per (token, head) of the fused qkv row: optional per-head RMSNorm, rotation,
// bf16 store of q, append of k and v to the cache.
__global__ void k_rope_store(RopeStoreArgs a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int heads = a.nh + 2 * a.nkv;
  const int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= a.M * heads) return;
  const int64_t m = w / heads;
  const int h = (int)(w - m * heads);
  const int64_t b = m / a.S, s = m - b * a.S, pos = (a.pos_dev ? *a.pos_dev : a.pos0) + s;
  const int d = a.d, half = d / 2;
  const float* src = a.qkv + m * (int64_t)heads * d + (int64_t)h * d;
  const bool is_q = h < a.nh, is_k = !is_q && h < a.nh + a.nkv;
  __nv_bfloat16* dst;
  if (is_q) dst = a.q_out + m * (int64_t)a.nh * d + (int64_t)h * d;
  else if (is_k) dst = a.k_cache + (((int64_t)b * a.nkv + (h - a.nh)) * a.Tmax + pos) * d;
  else dst = a.v_cache + (((int64_t)b * a.nkv + (h - a.nh - a.nkv)) * a.Tmax + pos) * d;
  if (!is_q && !is_k) {
    for (int e = lane; e < d; e += 32) dst[e] = __float2bfloat16_rn(src[e]);
    return;
  }
  const float* gamma = is_q ? a.q_gamma : a.k_gamma;
  float inv_rms = 1.f;
  if (gamma) {
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) ss += src[e] * src[e];
    ss = warp_sum(ss);
    inv_rms = 1.f / sqrtf(ss / (float)d + a.norm_eps);
  }
  for (int j = lane; j < half; j += 32) {
    float x1 = src[j], x2 = src[j + half];
    if (gamma) {
      const float g1 = a.norm_plus_one ? 1.f + gamma[j] : gamma[j];
      const float g2 = a.norm_plus_one ? 1.f + gamma[j + half] : gamma[j + half];
      x1 = x1 * inv_rms * g1;
      x2 = x2 * inv_rms * g2;
    }
    const float c = a.cos_t[pos * half + j], sn = a.sin_t[pos * half + j];
    dst[j] = __float2bfloat16_rn(c * x1 - sn * x2);
    dst[j + half] = __float2bfloat16_rn(c * x2 + sn * x1);
  }
}

// The same vectorised: one thread per eight elements of a head -- for q and k the rotation pairs
// (j .. j+3) and (j + d/2 .. j + d/2 + 3), for v eight consecutive values -- with 128-bit loads
// and 64-bit (q, k) or 128-bit (v) bf16 stores, contiguous across a warp.  The d/8 threads of a
// head are consecutive lanes of one warp (d a multiple of 8, at most 256), so the optional
// per-head RMSNorm is a shuffle reduction among them.
__global__ void k_rope_store_vec(RopeStoreArgs a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int heads = a.nh + 2 * a.nkv;
  const int d = a.d, half = d / 2, per_head = d / 8;
  const int64_t total = a.M * heads * per_head;
  const int64_t pos00 = a.pos_dev ? *a.pos_dev : a.pos0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t mh = i / per_head;
    const int t = (int)(i - mh * per_head);
    const int64_t m = mh / heads;
    const int h = (int)(mh - m * heads);
    const int64_t b = m / a.S, pos = pos00 + (m - b * a.S);
    const float* src = a.qkv + mh * d;
    if (h >= a.nh + a.nkv) {
      const float4 v0 = ((const float4*)src)[2 * t], v1 = ((const float4*)src)[2 * t + 1];
      __nv_bfloat16* dst = a.v_cache + ((b * a.nkv + (h - a.nh - a.nkv)) * a.Tmax + pos) * d + 8 * t;
      const __nv_bfloat162 p0 = __floats2bfloat162_rn(v0.x, v0.y), p1 = __floats2bfloat162_rn(v0.z, v0.w);
      const __nv_bfloat162 p2 = __floats2bfloat162_rn(v1.x, v1.y), p3 = __floats2bfloat162_rn(v1.z, v1.w);
      *(uint4*)dst = make_uint4(*(const uint32_t*)&p0, *(const uint32_t*)&p1, *(const uint32_t*)&p2, *(const uint32_t*)&p3);
      continue;
    }
    const int j = 4 * t;
    float4 x1 = *(const float4*)(src + j), x2 = *(const float4*)(src + j + half);
    const float* gamma = h < a.nh ? a.q_gamma : a.k_gamma;
    if (gamma) {
      float ss = x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w + x2.x * x2.x + x2.y * x2.y + x2.z * x2.z + x2.w * x2.w;
      const unsigned live = __activemask();  // whole heads are in or out of range together
      for (int o = per_head / 2; o; o >>= 1) ss += __shfl_xor_sync(live, ss, o);
      const float inv = 1.f / sqrtf(ss / (float)d + a.norm_eps);
      float4 g1 = *(const float4*)(gamma + j), g2 = *(const float4*)(gamma + j + half);
      if (a.norm_plus_one) {
        g1.x += 1.f; g1.y += 1.f; g1.z += 1.f; g1.w += 1.f;
        g2.x += 1.f; g2.y += 1.f; g2.z += 1.f; g2.w += 1.f;
      }
      x1.x = x1.x * inv * g1.x; x1.y = x1.y * inv * g1.y; x1.z = x1.z * inv * g1.z; x1.w = x1.w * inv * g1.w;
      x2.x = x2.x * inv * g2.x; x2.y = x2.y * inv * g2.y; x2.z = x2.z * inv * g2.z; x2.w = x2.w * inv * g2.w;
    }
    const float4 c = *(const float4*)(a.cos_t + pos * half + j), sn = *(const float4*)(a.sin_t + pos * half + j);
    __nv_bfloat16* dst = h < a.nh ? a.q_out + m * (int64_t)a.nh * d + (int64_t)h * d
                                  : a.k_cache + ((b * a.nkv + (h - a.nh)) * a.Tmax + pos) * d;
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(c.x * x1.x - sn.x * x2.x, c.y * x1.y - sn.y * x2.y);
    const __nv_bfloat162 l1 = __floats2bfloat162_rn(c.z * x1.z - sn.z * x2.z, c.w * x1.w - sn.w * x2.w);
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(c.x * x2.x + sn.x * x1.x, c.y * x2.y + sn.y * x1.y);
    const __nv_bfloat162 h1 = __floats2bfloat162_rn(c.z * x2.z + sn.z * x1.z, c.w * x2.w + sn.w * x1.w);
    *(uint2*)(dst + j) = make_uint2(*(const uint32_t*)&l0, *(const uint32_t*)&l1);
    *(uint2*)(dst + j + half) = make_uint2(*(const uint32_t*)&h0, *(const uint32_t*)&h1);
  }
}

// argmax over the vocabulary with the reference's ordering (total order on the bit patterns,
// last index wins ties), in two launches: every block folds a slice of one row into
// (key << 32 | index) and merges it into best[row] with a 64-bit atomic max, which is
// order-independent and therefore deterministic; a one-block kernel then publishes the
// tokens.  An optional soft-cap is written back to the logits first.
__global__ void k_argmax_part(float* logits, int64_t B, int64_t Vp, int parts, float softcap, unsigned long long* best_out,
                              uint32_t idx_off) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ unsigned long long sh[32];
  const int64_t b = blockIdx.y;
  const int64_t total = (int64_t)parts * Vp;
  const int64_t span = (total + gridDim.x - 1) / gridDim.x;
  const int64_t g0 = blockIdx.x * span, g1 = min(total, g0 + span);
  unsigned long long best = 0;
  for (int64_t g = g0 + threadIdx.x; g < g1; g += blockDim.x) {
    const int64_t part = g / Vp, i = g - part * Vp;
    float* p = logits + (part * B + b) * Vp + i;
    float v = *p;
    if (softcap > 0.f) { v = softcap * tanh_f(v / softcap); *p = v; }
    const uint32_t bits = __float_as_uint(v);
    const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    const unsigned long long q = ((unsigned long long)key << 32) | ((uint32_t)g + idx_off);
    best = q > best ? q : best;
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int o = 16; o; o >>= 1) {
    unsigned long long w = __shfl_xor_sync(0xffffffffu, best, o);
    best = w > best ? w : best;
  }
  if (lane == 0) sh[wid] = best;
  __syncthreads();
  if (wid == 0) {
    best = lane < nw ? sh[lane] : 0ull;
    for (int o = 16; o; o >>= 1) {
      unsigned long long w = __shfl_xor_sync(0xffffffffu, best, o);
      best = w > best ? w : best;
    }
    if (lane == 0 && g0 < g1) atomicMax(best_out + b, best);
  }
}
// publish the tokens, clear the merge slots for the next step and, when asked, count one
// more generated token and one more cached position
__global__ void k_argmax_finish(unsigned long long* best, int64_t B, uint32_t* tokens, uint32_t* history, int64_t hist_ld,
                                int64_t* count_dev, int64_t* pos_dev, int advance) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t count = *count_dev;
  for (int64_t b = threadIdx.x; b < B; b += blockDim.x) {
    const uint32_t t = (uint32_t)(best[b] & 0xFFFFFFFFull);
    tokens[b] = t;
    if (history) history[b * hist_ld + count] = t;
    best[b] = 0ull;
  }
  __syncthreads();
  if (threadIdx.x == 0 && advance) {
    *count_dev = count + 1;
    *pos_dev += 1;
  }
}

// One block per row: x[m, :] += addends of all ranks (rank order), then the row's RMSNorm.
template <int OUT_BF16>
__global__ void k_rmsnorm_reduce(PeerPush px, float* x, int64_t ldx, const float* gamma, float eps, int plus_one, int64_t H,
                                 void* out, int32_t* err) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float sh[32];
  const uint32_t e = *(volatile uint32_t*)px.epoch;  // the reduction the preceding kernel pushed
  const uint32_t par = e & 1u;
  if ((int)threadIdx.x < px.world) peer_wait_flag(px.flags[px.rank] + par * px.world + threadIdx.x, e, err);
  __syncthreads();
  const int64_t m = blockIdx.x;
  float* row = x + m * ldx;
  const float* slots = px.data[px.rank] + (int64_t)par * px.world * px.max_elems + m * H;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = row[i];
    for (int r = 0; r < px.world; ++r) acc += __ldcg(slots + (int64_t)r * px.max_elems + i);
    row[i] = acc;
    ss += acc * acc;
  }
  ss = block_sum(ss, sh);
  const float rms = sqrtf(ss / (float)H + eps);
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = plus_one ? 1.f + gamma[i] : gamma[i];
    const float v = row[i] / rms * g;  // this thread's own store above
    if (OUT_BF16) ((__nv_bfloat16*)out)[m * H + i] = __float2bfloat16_rn(v);
    else ((float*)out)[m * H + i] = v;
  }
}

// One block: push this rank's per-row candidates, collect every rank's, publish the tokens.
__global__ void k_argmax_finish_tp(PeerPush px, unsigned long long* best, int64_t B, uint32_t* tokens, uint32_t* history,
                                   int64_t hist_ld, int64_t* count_dev, int64_t* pos_dev, int advance, int32_t* err) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t e = *(volatile uint32_t*)px.epoch + 1u;
  const uint32_t par = e & 1u;
  const int64_t mine = ((int64_t)par * px.world + px.rank) * px.max_elems;
  for (int64_t b = threadIdx.x; b < B; b += blockDim.x) {
    const unsigned long long v = best[b];
    best[b] = 0ull;
    for (int r = 0; r < px.world; ++r) ((unsigned long long*)(px.data[r] + mine))[b] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < px.world; ++r)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(px.flags[r] + par * px.world + px.rank), "r"(e) : "memory");
    *(volatile uint32_t*)px.epoch = e;
  }
  if ((int)threadIdx.x < px.world) peer_wait_flag(px.flags[px.rank] + par * px.world + threadIdx.x, e, err);
  __syncthreads();
  const int64_t count = *count_dev;
  for (int64_t b = threadIdx.x; b < B; b += blockDim.x) {
    unsigned long long m = 0ull;
    for (int r = 0; r < px.world; ++r) {
      const unsigned long long v =
          __ldcg((const unsigned long long*)(px.data[px.rank] + ((int64_t)par * px.world + r) * px.max_elems) + b);
      m = v > m ? v : m;
    }
    const uint32_t t = (uint32_t)(m & 0xFFFFFFFFull);
    tokens[b] = t;
    if (history) history[b * hist_ld + count] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0 && advance) {
    *count_dev = count + 1;
    *pos_dev += 1;
  }
}

__global__ void k_to_bf16(const float* x, int64_t n, __nv_bfloat16* out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(x[i]);
}

// Pairs of N(mean, std) samples from a counter-based generator: splitmix64 of (seed, pair
// index) gives two 24-bit uniforms, Box-Muller turns them into two normals.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
template <typename T>
__global__ void k_randn(uint64_t seed, int64_t n, float mean, float std, T* out) {
  const int64_t pairs = (n + 1) / 2;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t h = mix64(seed ^ mix64((uint64_t)i));
    const float u1 = (float)((h >> 40) + 1) * (1.0f / 16777216.0f);       // (0, 1]
    const float u2 = (float)(h & 0xFFFFFFull) * (1.0f / 16777216.0f);     // [0, 1)
    const float r = sqrtf(-2.0f * logf(u1)) * std;
    float sn, cs;
    sincosf(6.283185307179586f * u2, &sn, &cs);
    out[2 * i] = (T)(mean + r * cs);
    if (2 * i + 1 < n) out[2 * i + 1] = (T)(mean + r * sn);
  }
}

}  // namespace

int k_launch_embed(cg_ctx* c, const uint32_t* tokens, int64_t tok_ld, int64_t tok_off, int64_t S, const void* table, int st,
                   int64_t vocab, int64_t M, int64_t H, float scale, float* out) {
  if (M == 0) return CG_OK;
  CG_CUDA(c, launch_kernel(c, k_embed, dim3((unsigned)M), dim3(256), 0, 1, tokens, tok_ld, tok_off, S, table, st, vocab, H,
                           scale, out, c->core->dev_err));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rmsnorm(cg_ctx* c, const float* x, int64_t ldx, const float* gamma, float eps, int plus_one, int64_t M,
                     int64_t H, void* out, int out_bf16) {
  if (M == 0) return CG_OK;
  // (up to 16 elements per thread stay in registers: 256 threads for rows of 4096, 512 for 8192)
  const int block = H > 4096 ? 512 : (H > 2048 ? 256 : 128);
  if (out_bf16) CG_CUDA(c, launch_kernel(c, k_rmsnorm<1>, dim3((unsigned)M), dim3(block), 0, 1, x, ldx, gamma, eps, plus_one, H, out));
  else CG_CUDA(c, launch_kernel(c, k_rmsnorm<0>, dim3((unsigned)M), dim3(block), 0, 1, x, ldx, gamma, eps, plus_one, H, out));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rmsnorm_add(cg_ctx* c, const float* y, const float* gamma, float eps, int plus_one, int64_t M, int64_t H,
                         float* x) {
  if (M == 0) return CG_OK;
  const int block = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  CG_CUDA(c, launch_kernel(c, k_rmsnorm<2>, dim3((unsigned)M), dim3(block), 0, 1, y, H, gamma, eps, plus_one, H, (void*)x));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rmsnorm_add_norm(cg_ctx* c, const float* y, const float* g1, const float* g2, float eps, int plus_one, int64_t M,
                              int64_t H, float* x, __nv_bfloat16* out) {
  if (M == 0) return CG_OK;
  const int block = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  CG_CUDA(c, launch_kernel(c, k_rmsnorm_add_norm, dim3((unsigned)M), dim3(block), 0, 1, y, g1, g2, eps, plus_one, H, x, out));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_add_bf16_norm(cg_ctx* c, const __nv_bfloat16* t, const float* g, float eps, int plus_one, int64_t M, int64_t H,
                           float* x, __nv_bfloat16* out) {
  if (M == 0) return CG_OK;
  if (H % 2) return fail(c, CG_ERR_UNSUPPORTED, "add + norm: the row length must be even");
  const int block = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  CG_CUDA(c, launch_kernel(c, k_add_bf16_norm, dim3((unsigned)M), dim3(block), 0, 1, t, g, eps, plus_one, H, x, out));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_act_mul(cg_ctx* c, const float* gu, int64_t M, int64_t F, int act, __nv_bfloat16* out) {
  if (M == 0 || F == 0) return CG_OK;
  dim3 grid((unsigned)std::min<int64_t>((F / 4 + 255) / 256 + 1, 64), (unsigned)M);
  CG_CUDA(c, launch_kernel(c, k_act_mul, grid, dim3(256), 0, 1, gu, F, act, out));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rope_tables(cg_ctx* c, float theta, int64_t T, int64_t d, float* cos_t, float* sin_t) {
  const int64_t n = T * (d / 2);
  if (n == 0) return CG_OK;
  const float two_over_d = 2.0f / (float)d;
  k_rope_tables<<<grid_for(n, 256), 256, 0, c->core->stream>>>(theta, T, d / 2, two_over_d, cos_t, sin_t);
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rope_tables_scaled(cg_ctx* c, float theta, const RopeScaling& rs, int64_t T, int64_t d, float* cos_t, float* sin_t) {
  if (rs.kind == 0) return k_launch_rope_tables(c, theta, T, d, cos_t, sin_t);
  if (rs.kind != 1 && rs.kind != 2) return fail(c, CG_ERR_INVALID, "rope scaling: kind must be 0 (none), 1 (llama3) or 2 (yarn)");
  if (rs.factor <= 0.f || rs.original_max_pos <= 0) return fail(c, CG_ERR_INVALID, "rope scaling: factor and original_max_pos must be positive");
  if (rs.kind == 1 && rs.high_freq_factor == rs.low_freq_factor) return fail(c, CG_ERR_INVALID, "rope scaling: high and low frequency factors coincide");
  const int64_t n = T * (d / 2);
  if (n == 0) return CG_OK;
  float low = 0.f, high = 1.f, mscale = 1.f;
  if (rs.kind == 2) {
    // find_correction_range and rope_yarn_get_mscale (rope.rs:100-128), in f32 like the reference
    const float two_pi = 2.0f * 3.14159265358979323846f;
    auto corr = [&](float rot) { return ((float)d * logf((float)rs.original_max_pos / (rot * two_pi))) / (2.f * logf(theta)); };
    low = corr(rs.beta_fast);
    high = corr(rs.beta_slow);
    if (high == low) return fail(c, CG_ERR_INVALID, "rope scaling: empty yarn correction range");
    mscale = rs.factor <= 1.0f ? 1.0f : 0.1f * logf(rs.factor) + 1.0f;
  }
  k_rope_tables_scaled<<<grid_for(n, 256), 256, 0, c->core->stream>>>(theta, rs, low, high, mscale, T, d / 2, 2.0f / (float)d, cos_t, sin_t);
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rope_store(cg_ctx* c, const RopeStoreArgs& a) {
  const int64_t warps = a.M * (a.nh + 2 * a.nkv);
  if (warps == 0) return CG_OK;
  if (a.d % 8 == 0 && ((!a.q_gamma && !a.k_gamma) || (a.q_gamma && a.k_gamma && a.d <= 256 && (256 % a.d) == 0))) {
    const int64_t items = warps * (a.d / 8);
    CG_CUDA(c, launch_kernel(c, k_rope_store_vec, dim3(grid_for(items, 256, 148 * 32)), dim3(256), 0, 1, a));
    CG_LAUNCHED(c);
    return CG_OK;
  }
  const int block = 256;
  const int64_t blocks = (warps * 32 + block - 1) / block;
  CG_CUDA(c, launch_kernel(c, k_rope_store, dim3((unsigned)blocks), dim3(block), 0, 1, a));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_argmax(cg_ctx* c, float* logits, int64_t B, int64_t Vp, int parts, float softcap, uint32_t* tokens,
                    uint32_t* history, int64_t hist_ld, int64_t* count_dev, int64_t* pos_dev, int advance,
                    unsigned long long* best) {
  if (B == 0) return CG_OK;
  const int64_t total = (int64_t)parts * Vp;
  const unsigned chunks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(64, total / 1024));
  CG_CUDA(c, launch_kernel(c, k_argmax_part, dim3(chunks, (unsigned)B), dim3(256), 0, 1, logits, B, Vp, parts, softcap, best,
                           (uint32_t)0));
  CG_LAUNCHED(c);
  CG_CUDA(c, launch_kernel(c, k_argmax_finish, dim3(1), dim3(64), 0, 1, best, B, tokens, history, hist_ld, count_dev, pos_dev,
                           advance));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_rmsnorm_reduce(cg_ctx* c, const PeerPush& px, float* x, int64_t ldx, const float* gamma, float eps, int plus_one,
                            int64_t M, int64_t H, void* out, int out_bf16) {
  if (M == 0) return CG_OK;
  if (M * H > px.max_elems) return fail(c, CG_ERR_INVALID, "rmsnorm_reduce: rows do not fit the exchange area");
  const int block = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (out_bf16)
    CG_CUDA(c, launch_kernel(c, k_rmsnorm_reduce<1>, dim3((unsigned)M), dim3(block), 0, 1, px, x, ldx, gamma, eps, plus_one, H, out,
                             c->core->dev_err));
  else
    CG_CUDA(c, launch_kernel(c, k_rmsnorm_reduce<0>, dim3((unsigned)M), dim3(block), 0, 1, px, x, ldx, gamma, eps, plus_one, H, out,
                             c->core->dev_err));
  CG_LAUNCHED(c);
  return CG_OK;
}

int k_launch_argmax_tp(cg_ctx* c, const PeerPush& px, float* logits, int64_t B, int64_t Vp, float softcap, uint32_t* tokens,
                       uint32_t* history, int64_t hist_ld, int64_t* count_dev, int64_t* pos_dev, int advance,
                       unsigned long long* best) {
  if (B == 0) return CG_OK;
  if (2 * B > px.max_elems) return fail(c, CG_ERR_INVALID, "argmax: rows do not fit the exchange area");
  const unsigned chunks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(64, Vp / 1024));
  CG_CUDA(c, launch_kernel(c, k_argmax_part, dim3(chunks, (unsigned)B), dim3(256), 0, 1, logits, B, Vp, 1, softcap, best,
                           (uint32_t)((int64_t)px.rank * Vp)));
  CG_LAUNCHED(c);
  CG_CUDA(c, launch_kernel(c, k_argmax_finish_tp, dim3(1), dim3(64), 0, 1, px, best, B, tokens, history, hist_ld, count_dev, pos_dev,
                           advance, c->core->dev_err));
  CG_LAUNCHED(c);
  return CG_OK;
}

// waits on a word of the error block that stays zero
__global__ void k_probe_wait(int32_t* err) { peer_wait_flag((const uint32_t*)(err + 8), 1u, err); }

int k_launch_to_bf16(cg_ctx* c, const float* x, int64_t n, __nv_bfloat16* out) {
  if (n == 0) return CG_OK;
  CG_CUDA(c, launch_kernel(c, k_to_bf16, dim3(grid_for(n, 256)), dim3(256), 0, 1, x, n, out));
  CG_LAUNCHED(c);
  return CG_OK;
}

}  // namespace cg

using namespace cg;

// --------------------------------------------------------------- public fused entry points

extern "C" {

int32_t cg_fused_rmsnorm(cg_ctx* c, const cg_tensor* x, const cg_tensor* gamma, float eps, int32_t plus_one, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !gamma || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32 || gamma->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "rmsnorm wants F32 tensors");
  if (x->rank < 1 || gamma->numel() != x->dims[x->rank - 1]) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  Hold xc, gc, r;
  CG_TRY(as_contiguous_f32(c, x, &xc.t));
  CG_TRY(as_contiguous_f32(c, gamma, &gc.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
  const int64_t H = x->dims[x->rank - 1];
  const int64_t M = H ? x->numel() / H : 0;
  if (M > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "too many rows");
  CG_TRY(k_launch_rmsnorm(c, (const float*)xc.t->data(), H, (const float*)gc.t->data(), eps, plus_one, M, H, r.t->data(), 0));
  *out = r.take();
  return CG_OK;
}

int32_t cg_fused_softmax(cg_ctx* c, const cg_tensor* x, float softcap, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "softmax wants an F32 tensor");
  if (x->rank < 1) return fail(c, CG_ERR_SHAPE, "softmax of a rank-0 tensor");
  Hold xc, r;
  CG_TRY(as_contiguous_f32(c, x, &xc.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
  const int64_t n = x->dims[x->rank - 1];
  const int64_t rows = n ? x->numel() / n : 0;
  if (rows > 2147483647ll) return fail(c, CG_ERR_UNSUPPORTED, "too many rows");
  if (rows) {
    const int block = n > 4096 ? 512 : (n > 2048 ? 256 : (n >= 256 ? 128 : 64));
    k_softmax<<<(unsigned)rows, block, 0, c->core->stream>>>((const float*)xc.t->data(), n, softcap, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_fused_act_mul(cg_ctx* c, const cg_tensor* gate, const cg_tensor* up, int32_t act, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !gate || !up || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (gate->tag != CG_F32 || up->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "act_mul wants F32 tensors");
  if (gate->rank != up->rank) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  for (int i = 0; i < gate->rank; ++i)
    if (gate->dims[i] != up->dims[i]) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  if (act != 0 && act != 1) return fail(c, CG_ERR_INVALID, "unknown activation");
  Hold g, u, r;
  CG_TRY(as_contiguous_f32(c, gate, &g.t));
  CG_TRY(as_contiguous_f32(c, up, &u.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, gate->dims, gate->rank, &r.t));
  const int64_t n = r.t->numel();
  if (n) {
    const bool aligned = ((((uintptr_t)g.t->data()) | ((uintptr_t)u.t->data()) | ((uintptr_t)r.t->data())) & 15) == 0;
    if ((n & 3) == 0 && aligned)
      k_act_mul_f32_vec<<<grid_for(n / 8 + 1, 256, 148 * 32), 256, 0, c->core->stream>>>(
          (const float4*)g.t->data(), (const float4*)u.t->data(), n / 4, act, (float4*)r.t->data());
    else
      k_act_mul_f32<<<grid_for(n, 256), 256, 0, c->core->stream>>>((const float*)g.t->data(), (const float*)u.t->data(), n,
                                                                  act, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_fused_rope(cg_ctx* c, const cg_tensor* x, float theta, int64_t pos0, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "rope wants an F32 tensor");
  if (x->rank != 4 || (x->dims[3] & 1) || pos0 < 0) return fail(c, CG_ERR_SHAPE, "rope wants [b, heads, s, d] with even d");
  const int64_t S = x->dims[2], d = x->dims[3], T = pos0 + S;
  Hold xc, r, ct, sn;
  CG_TRY(as_contiguous_f32(c, x, &xc.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
  int64_t td[2] = {T, d / 2};
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &ct.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &sn.t));
  CG_TRY(k_launch_rope_tables(c, theta, T, d, (float*)ct.t->data(), (float*)sn.t->data()));
  const int64_t n = r.t->numel();
  if (n) {
    const bool aligned = ((((uintptr_t)xc.t->data()) | ((uintptr_t)r.t->data()) | ((uintptr_t)ct.t->data()) | ((uintptr_t)sn.t->data())) & 15) == 0;
    if (d % 8 == 0 && aligned)
      k_rope_apply_vec<<<grid_for(n / 8, 256, 148 * 32), 256, 0, c->core->stream>>>(
          (const float*)xc.t->data(), (const float*)ct.t->data(), (const float*)sn.t->data(), S, d, pos0, n / 8, (float*)r.t->data());
    else
      k_rope_apply<<<grid_for(n, 256), 256, 0, c->core->stream>>>((const float*)xc.t->data(), (const float*)ct.t->data(),
                                                                 (const float*)sn.t->data(), S, d, pos0, n,
                                                                 (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_linear(cg_ctx* c, const cg_tensor* x, const cg_tensor* w, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !w || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32 || w->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "linear wants F32 tensors");
  if (x->rank < 1 || w->rank != 2 || x->dims[x->rank - 1] != w->dims[1]) return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  const int64_t K = w->dims[1], N = w->dims[0];
  const int64_t M = K ? x->numel() / K : 0;
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = N;
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, od, x->rank, &r.t));
  if (r.t->numel() == 0) { *out = r.take(); return CG_OK; }
  if (K == 0) {
    CG_CUDA(c, cudaMemsetAsync(r.t->data(), 0, (size_t)r.t->numel() * 4, c->core->stream));
    *out = r.take();
    return CG_OK;
  }
  const bool tc = c->opt_gemm == 0 && w->storage == ST_BF16 && w->contiguous() && K % 8 == 0 &&
                  ((uintptr_t)w->data() % 16 == 0);
  if (tc) {
    Hold xc, xb;
    CG_TRY(as_contiguous(c, x, &xc.t));
    const __nv_bfloat16* xp;
    CG_TRY(bf16_operand(c, xc.t, M, K, K, 1, &xb.t, &xp));
    CG_TRY(gemm_tc(c, xp, K, (const __nv_bfloat16*)w->data(), K, r.t->data(), N, nullptr, M, N, K, 0, 0, nullptr));
  } else {
    // [1, M, K] x [1, K, N] through strided views, like linear_b_param's transpose + reshape
    Hold xc;
    CG_TRY(as_contiguous(c, x, &xc.t));
    Hold xv(new_view(xc.t)), wv(new_view(w)), rv(new_view(r.t));
    xv.t->rank = 2; xv.t->dims[0] = M; xv.t->dims[1] = K; xv.t->strides[0] = K; xv.t->strides[1] = 1;
    wv.t->rank = 2; wv.t->dims[0] = K; wv.t->dims[1] = N; wv.t->strides[0] = w->strides[1]; wv.t->strides[1] = w->strides[0];
    rv.t->rank = 2; rv.t->dims[0] = M; rv.t->dims[1] = N; rv.t->strides[0] = N; rv.t->strides[1] = 1;
    CG_TRY(gemm_simt(c, xv.t, wv.t, rv.t));
  }
  *out = r.take();
  return CG_OK;
}

int32_t cg_linear_glu(cg_ctx* c, const cg_tensor* x, const cg_tensor* w, int32_t act, cg_tensor** out) {
  CG_LAZY_EAGER_SCOPE(c);
  if (!c || !x || !w || !out) return fail(c, CG_ERR_INVALID, "null argument");
  if (x->tag != CG_F32 || w->tag != CG_F32) return fail(c, CG_ERR_DTYPE, "linear_glu wants F32 tensors");
  if (act != 0 && act != 1) return fail(c, CG_ERR_INVALID, "linear_glu: act is 0 (silu) or 1 (tanh gelu)");
  if (x->rank < 1 || w->rank != 2 || x->dims[x->rank - 1] != w->dims[1] || (w->dims[0] & 1))
    return fail(c, CG_ERR_SHAPE, "Shape mismatch in operation");
  const int64_t K = w->dims[1], F = w->dims[0] / 2;
  if (w->storage != ST_BF16 || !w->contiguous() || K == 0 || K % 8 || ((uintptr_t)w->data() % 16))
    return fail(c, CG_ERR_UNSUPPORTED, "linear_glu wants a contiguous bf16-stored weight [2F, K] with K a multiple of 8");
  const int64_t M = x->numel() / K;
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = F;
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, od, x->rank, &r.t));
  if (r.t->numel() == 0) { *out = r.take(); return CG_OK; }
  Hold xc, xb;
  CG_TRY(as_contiguous(c, x, &xc.t));
  const __nv_bfloat16* xp;
  CG_TRY(bf16_operand(c, xc.t, M, K, K, 1, &xb.t, &xp));
  CG_TRY(gemm_tc_pair(c, xp, K, (const __nv_bfloat16*)w->data(), K, (__nv_bfloat16*)r.t->data(), F, M, F, K, act));
  *out = r.take();
  return CG_OK;
}

int32_t cg_randn(cg_ctx* c, const int64_t* dims, int32_t rank, uint64_t seed, float mean, float std, cg_tensor** out) {
  if (!c || !out || rank < 0 || rank > CG_MAX_RANK || (rank && !dims)) return fail(c, CG_ERR_INVALID, "bad argument");
  // same storage rule as an upload: matrices are kept in bf16 by a bf16-precision context
  const int st = c->precision == CG_PREC_BF16 && rank >= 2 ? ST_BF16 : ST_F32;
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, st, dims, rank, &r.t));
  const int64_t n = r.t->numel();
  if (n) {
    const unsigned grid = grid_for((n + 1) / 2, 256);
    if (st == ST_BF16) k_randn<<<grid, 256, 0, c->core->stream>>>(seed, n, mean, std, (__nv_bfloat16*)r.t->data());
    else k_randn<<<grid, 256, 0, c->core->stream>>>(seed, n, mean, std, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

}  // extern "C"

extern "C" int32_t cg_probe_wait_timeout(cg_ctx* c) {
  if (!c) return CG_ERR_INVALID;
  cg::k_probe_wait<<<1, 1, 0, c->core->stream>>>(c->core->dev_err);
  CG_LAUNCHED(c);
  return CG_OK;
}

extern "C" int32_t cg_rope_tables(cg_ctx* c, float theta, int32_t kind, float factor, float low_freq_factor, float high_freq_factor,
                                  float beta_fast, float beta_slow, int32_t original_max_pos, int64_t T, int64_t d,
                                  cg_tensor** cos_out, cg_tensor** sin_out) {
  if (!c || !cos_out || !sin_out || T < 0 || d < 2 || d % 2) return fail(c, CG_ERR_INVALID, "rope tables: bad argument");
  RopeScaling rs;
  rs.kind = kind; rs.factor = factor; rs.low_freq_factor = low_freq_factor; rs.high_freq_factor = high_freq_factor;
  rs.beta_fast = beta_fast; rs.beta_slow = beta_slow; rs.original_max_pos = original_max_pos;
  int64_t td[2] = {T, d / 2};
  Hold ct, sn;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &ct.t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &sn.t));
  CG_TRY(k_launch_rope_tables_scaled(c, theta, rs, T, d, (float*)ct.t->data(), (float*)sn.t->data()));
  *cos_out = ct.take();
  *sin_out = sn.take();
  return CG_OK;
}
