// lazy.cu — deferred evaluation of the trait methods with pattern fusion.
//
// The interpreter drives a backend one primitive at a time (catgrad/src/interpreter/tensor_op.rs:9-42
// walked by catgrad/src/abstract_interpreter/eval.rs:18-77): an RMSNorm arrives as a dozen calls, a
// softmax as seven, an attention core as more than thirty with an S x S score tensor in between.
// With the "lazy" option the same calls are RECORDED instead of run: every recorded call returns
// a tensor handle that has its shape and dtype but no contents yet.  When contents are needed
// (to_vec, compare, a call that is not recorded, cg_sync) the recorded nodes run in order, except
// that the chains the reference's stdlib and model graphs are made of are recognised and replaced
// by one fused kernel each:
//
//   rmsnorm          catgrad-llm/src/helpers.rs:120-145  (and the (1 + gamma) form of models/gemma3.rs:60-68)
//   softmax          catgrad/src/stdlib/nn/mod.rs:162-171
//   silu(g) * u      nn/mod.rs:130-148 with the product of models/llama.rs:27; gelu(g) * u (nn/mod.rs:151-160, models/gemma3.rs:28)
//   rope             catgrad-llm/src/helpers.rs:202-221 (tables given as tensors)
//   attention core   models/llama.rs:97-108: q k^T / sqrt(d) + causal mask -> softmax -> p v, seen
//                    through repeat_kv (helpers.rs:147-161) and the rotation of k, so the S x S
//                    scores, the mask and the repeated keys / values never exist
//
// Everything else runs exactly as in eager mode, through the same entry points.  A node inside a
// recognised chain is skipped only if nobody else needs its value: no other node reads it and the
// caller holds no handle to it.  Views (broadcast, transpose, slice, layout-compatible reshape) of
// pending tensors are recorded too, as aliases that cost nothing when they run.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>
#include <unordered_set>

#include "kernels.h"

namespace cg {

enum LzOp : int {
  LZ_BROADCAST = 0, LZ_TRANSPOSE, LZ_SLICE, LZ_RESHAPE,  // aliases (same order as LazyView)
  LZ_RESHAPE_COPY, LZ_CAST, LZ_ADD, LZ_SUB, LZ_MUL, LZ_DIV, LZ_POW, LZ_LT, LZ_NEG, LZ_MAX, LZ_SUM, LZ_MATMUL, LZ_CONCAT,
  LZ_ARANGE
};
enum Fuse : int { F_NONE = 0, F_RMSNORM, F_SOFTMAX, F_SILU_MUL, F_ROPE, F_ATTENTION };

struct LazyNode {
  int op = 0;
  cg_tensor* in[2] = {nullptr, nullptr};  // retained while the node is pending
  int nin = 0;
  int64_t a[CG_MAX_RANK + 2] = {0};       // op arguments
  int na = 0;
  cg_tensor* out = nullptr;               // the handle that stands for the result (not retained)
  bool dead = false;                      // the result was dropped before it was needed
  int index = 0;
  // set by the matcher
  int fuse = F_NONE;                      // this node is the root of a recognised chain
  LazyNode* claimed = nullptr;            // this node is inside the chain rooted there
  // what the fused kernel needs (meaning depends on `fuse`)
  cg_tensor* m_t[4] = {nullptr, nullptr, nullptr, nullptr};
  const float* m_p[2] = {nullptr, nullptr};
  float m_f = 0.f;
  int64_t m_i[4] = {0, 0, 0, 0};
};

namespace {

bool is_alias(int op) { return op <= LZ_RESHAPE; }

LazyNode* producer(const cg_tensor* t) { return t ? t->node : nullptr; }

cg_tensor* pending_tensor(cg_ctx* c, int tag, const int64_t* dims, int rank) {
  auto* t = new cg_tensor();
  t->ctx = c;
  t->tag = tag;
  t->storage = tag == CG_F32 ? ST_F32 : ST_U32;
  t->rank = rank;
  int64_t n = 1;
  for (int i = rank - 1; i >= 0; --i) {
    t->dims[i] = dims[i];
    t->strides[i] = n;
    n *= dims[i];
  }
  return t;
}

LazyNode* add_node(cg_ctx* c, int op, cg_tensor* out, const cg_tensor* in0, const cg_tensor* in1) {
  auto* n = new LazyNode();
  n->op = op;
  n->out = out;
  n->index = (int)c->lazy_nodes.size();
  const cg_tensor* ins[2] = {in0, in1};
  for (const cg_tensor* t : ins) {
    if (!t) continue;
    auto* m = const_cast<cg_tensor*>(t);
    m->rc++;
    m->lazy_uses++;
    n->in[n->nin++] = m;
  }
  out->node = n;
  c->lazy_nodes.push_back(n);
  c->lazy_recorded++;
  return n;
}

bool same_shape(const cg_tensor* a, const cg_tensor* b) {
  if (a->rank != b->rank) return false;
  for (int i = 0; i < a->rank; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

// Handles the caller holds: references that are not recorded nodes reading the tensor.
int user_refs(const cg_tensor* t) { return (int)t->rc - t->lazy_uses; }

void drop_inputs(LazyNode* n) {
  for (int i = 0; i < n->nin; ++i) {
    cg_tensor* t = n->in[i];
    n->in[i] = nullptr;
    if (!t) continue;
    t->lazy_uses--;
    release(t);
  }
  n->nin = 0;
}

// The pending handle `out` receives the contents of the freshly computed `res`.
// (Results of the entry points are contiguous, which is the layout the handle was given when the
// call was recorded and relative to which views of it were recorded; only the offset can differ.)
void adopt(cg_tensor* out, cg_tensor* res) {
  out->buf = res->buf;
  out->storage = res->storage;
  out->offset = res->offset;
  out->node = nullptr;
}

// ------------------------------------------------------------------------------------------
// fused kernels used only from here

// out = cos * x + sin * rotate_half(x) with the tables given as tensors: x [b, h, S, d] with
// arbitrary strides over b, h, S (unit stride over d), cos / sin rows of d floats `ld` apart for
// positions 0..S, out contiguous.  One thread per rotation pair.
__global__ void k_rope_tab(const float* x, int64_t sb, int64_t sh, int64_t ss, const float* cos_t, const float* sin_t, int64_t ld,
                           int64_t H, int64_t S, int64_t d, int64_t n_pairs, float* out) {
  const int64_t half = d / 2;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_pairs; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t j = i % half, r = i / half;  // r = (b * H + h) * S + s
    const int64_t s = r % S, bh = r / S, h = bh % H, b = bh / H;
    const float* xr = x + b * sb + h * sh + s * ss;
    const float x1 = xr[j], x2 = xr[j + half];
    const float c1 = cos_t[s * ld + j], c2 = cos_t[s * ld + j + half], s1 = sin_t[s * ld + j], s2 = sin_t[s * ld + j + half];
    float* o = out + r * d;
    o[j] = c1 * x1 + s1 * -x2;
    o[j + half] = c2 * x2 + s2 * x1;
  }
}

// f32 causal attention for the exact-parity path: out[b, h, i, :] = softmax_j(q_i . k_j * scale, j <= i) v_j.
// q [b, nh, S, d], k / v [b, nkv, S, d] with arbitrary strides over the first three axes (unit
// stride over d), head h reads kv head h / rep; out contiguous [b, nh, S, d].  A block owns 32
// query rows of one head; keys and values pass through shared memory 32 at a time; every sum is
// f32 with an online softmax, exp through expf.
template <int D>
__global__ void __launch_bounds__(128) k_attn_f32(const float* q, const int64_t* qs, const float* k, const int64_t* ks, const float* v,
                                                   const int64_t* vs, int64_t S, int rep, float scale, int scale_is_div, int out_bshd,
                                                   float* out) {
  extern __shared__ float attn_smem[];
  float (*qsm)[D + 1] = (float (*)[D + 1])attn_smem;
  float (*ksm)[D + 1] = qsm + 32;
  float (*vsm)[D + 1] = ksm + 32;
  float (*psm)[33] = (float (*)[33])(vsm + 32);
  const int h = blockIdx.y, b = blockIdx.z, q0 = blockIdx.x * 32;
  const int ty = threadIdx.x >> 2, tx = threadIdx.x & 3;  // query row, quarter
  const int64_t qi = q0 + ty;
  const float* qb = q + b * qs[0] + h * qs[1];
  const float* kb = k + b * ks[0] + (h / rep) * ks[1];
  const float* vb = v + b * vs[0] + (h / rep) * vs[1];
  for (int e = threadIdx.x; e < 32 * D; e += 128) {
    const int r = e / D, col = e - r * D;
    qsm[r][col] = q0 + r < S ? qb[(q0 + r) * qs[2] + col] : 0.f;
  }
  constexpr int CPT = D / 4;  // output columns per thread
  float o[CPT];
#pragma unroll
  for (int i = 0; i < CPT; ++i) o[i] = 0.f;
  float m = -3.4028234663852886e38f, l = 0.f;
  const int last_tile = (int)((min((int64_t)q0 + 31, S - 1)) / 32);
  for (int t = 0; t <= last_tile; ++t) {
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * D; e += 128) {
      const int r = e / D, col = e - r * D;
      const int64_t kj = (int64_t)t * 32 + r;
      ksm[r][col] = kj < S ? kb[kj * ks[2] + col] : 0.f;
      vsm[r][col] = kj < S ? vb[kj * vs[2] + col] : 0.f;
    }
    __syncthreads();
    // scores of this thread's 8 keys
    float sc[8];
    float mx = -3.4028234663852886e38f;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int kr = tx * 8 + jj;
      const int64_t kj = (int64_t)t * 32 + kr;
      float acc = 0.f;
      for (int col = 0; col < D; ++col) acc += qsm[ty][col] * ksm[kr][col];
      acc = scale_is_div ? acc / scale : acc * scale;
      const bool live = kj <= qi && kj < S;
      sc[jj] = live ? acc : -3.4028234663852886e38f;
      mx = fmaxf(mx, sc[jj]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mnew = fmaxf(m, mx);
    const float corr = expf(m - mnew);
    float sum = 0.f;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int64_t kj = (int64_t)t * 32 + tx * 8 + jj;
      const float p = (kj <= qi && kj < S) ? expf(sc[jj] - mnew) : 0.f;
      psm[ty][tx * 8 + jj] = p;
      sum += p;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l = l * corr + sum;
    m = mnew;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < CPT; ++i) o[i] *= corr;
    for (int kr = 0; kr < 32; ++kr) {
      const float p = psm[ty][kr];
#pragma unroll
      for (int i = 0; i < CPT; ++i) o[i] += p * vsm[kr][tx * CPT + i];
    }
  }
  if (qi < S) {
    // [b, nh, S, d], or [b, S, nh, d]: the layout the graph's transpose(1, 2) + reshape asks for next
    float* orow = out + (out_bshd ? (((int64_t)b * S + qi) * gridDim.y + h) : (((int64_t)b * gridDim.y + h) * S + qi)) * D + tx * CPT;
#pragma unroll
    for (int i = 0; i < CPT; ++i) orow[i] = o[i] / l;
  }
}

// ------------------------------------------------------------------------------------------
// matching helpers

bool scalar_f32(const cg_tensor* t, float* v) {
  if (!t || t->node || !t->has_scalar || t->tag != CG_F32) return false;
  memcpy(v, &t->scalar_bits, 4);
  return true;
}
bool scalar_is(const cg_tensor* t, float want, float rel = 0.f) {
  float v;
  if (!scalar_f32(t, &v)) return false;
  return rel > 0.f ? fabsf(v - want) <= rel * fabsf(want) : v == want;
}
// the node that produces t, if it is still pending, has the given op and is not already inside a chain
LazyNode* node_of(const cg_tensor* t, int op) {
  LazyNode* n = producer(t);
  return n && n->op == op && !n->claimed && !n->fuse ? n : nullptr;
}
// t = slice(x, dim, start, len) (as a recorded alias, or as a view of a concrete x)
bool is_slice_of(const cg_tensor* t, const cg_tensor* x, int dim, int64_t start, int64_t len, std::vector<LazyNode*>* chain) {
  if (LazyNode* n = node_of(t, LZ_SLICE)) {
    if (n->in[0] == x && n->a[0] == dim && n->a[1] == start && n->a[2] == len) { chain->push_back(n); return true; }
    return false;
  }
  if (t->node || x->node) return false;
  if (t->buf != x->buf || t->rank != x->rank || t->offset != x->offset + start * x->strides[dim]) return false;
  for (int i = 0; i < x->rank; ++i)
    if (t->strides[i] != x->strides[i] || t->dims[i] != (i == dim ? len : x->dims[i])) return false;
  return true;
}
// t is a concrete contiguous f32 vector of n elements seen through a broadcast (all other strides 0)
const float* broadcast_vector(const cg_tensor* t, int64_t n) {
  if (!t || t->node || t->tag != CG_F32 || t->storage != ST_F32 || t->rank < 1) return nullptr;
  if (t->dims[t->rank - 1] != n || (n > 1 && t->strides[t->rank - 1] != 1)) return nullptr;
  for (int i = 0; i < t->rank - 1; ++i)
    if (t->dims[i] != 1 && t->strides[i] != 0) return nullptr;
  return (const float*)t->data();
}

// rmsnorm: root = mul(raw, gamma_b) or mul(raw, add(one, gamma_b)) with
// raw = div(x, broadcast(pow(add(div(sum(mul(x, x)), n), eps), 0.5)))
bool match_rmsnorm(LazyNode* root, std::vector<LazyNode*>* interior) {
  if (root->op != LZ_MUL) return false;
  LazyNode* raw = node_of(root->in[0], LZ_DIV);
  if (!raw) return false;
  cg_tensor* x = raw->in[0];
  if (x->tag != CG_F32 || x->rank < 1) return false;
  const int64_t H = x->dims[x->rank - 1];
  LazyNode* bden = node_of(raw->in[1], LZ_BROADCAST);
  if (!bden) return false;
  LazyNode* rms = node_of(bden->in[0], LZ_POW);
  if (!rms || !scalar_is(rms->in[1], 0.5f)) return false;
  LazyNode* plus = node_of(rms->in[0], LZ_ADD);
  float eps;
  if (!plus || !scalar_f32(plus->in[1], &eps)) return false;
  LazyNode* mean = node_of(plus->in[0], LZ_DIV);
  if (!mean || !scalar_is(mean->in[1], (float)H)) return false;
  LazyNode* ssum = node_of(mean->in[0], LZ_SUM);
  if (!ssum) return false;
  LazyNode* sq = node_of(ssum->in[0], LZ_MUL);
  if (!sq || sq->in[0] != x || sq->in[1] != x) return false;
  int plus_one = 0;
  const float* gamma = broadcast_vector(root->in[1], H);
  LazyNode* gadd = nullptr;
  if (!gamma) {
    gadd = node_of(root->in[1], LZ_ADD);
    if (!gadd || !scalar_is(gadd->in[0], 1.0f)) return false;
    gamma = broadcast_vector(gadd->in[1], H);
    if (!gamma) return false;
    plus_one = 1;
  }
  if (!same_shape(root->out, x)) return false;
  *interior = {sq, ssum, mean, plus, rms, bden, raw};
  if (gadd) interior->push_back(gadd);
  root->m_t[0] = x;
  root->m_p[0] = gamma;
  root->m_f = eps;
  root->m_i[0] = plus_one;
  return true;
}

// softmax: root = div(ex, broadcast(sum(ex))), ex = pow(e, sub(x, broadcast(max(x))))
bool match_softmax(LazyNode* root, std::vector<LazyNode*>* interior, cg_tensor** x_out) {
  if (root->op != LZ_DIV) return false;
  LazyNode* ex = node_of(root->in[0], LZ_POW);
  LazyNode* bsum = node_of(root->in[1], LZ_BROADCAST);
  if (!ex || !bsum) return false;
  LazyNode* s = node_of(bsum->in[0], LZ_SUM);
  if (!s || s->in[0] != ex->out) return false;
  if (!scalar_is(ex->in[0], 2.7182817f, 1e-6f)) return false;
  LazyNode* sub = node_of(ex->in[1], LZ_SUB);
  if (!sub) return false;
  cg_tensor* x = sub->in[0];
  LazyNode* bmax = node_of(sub->in[1], LZ_BROADCAST);
  if (!bmax) return false;
  LazyNode* mx = node_of(bmax->in[0], LZ_MAX);
  if (!mx || mx->in[0] != x || x->tag != CG_F32) return false;
  *interior = {mx, bmax, sub, ex, s, bsum};
  *x_out = x;
  return true;
}

// silu(g) * u: root = mul(mul(g, div(one, add(one, pow(e, neg(g))))), u)
bool match_silu_mul(LazyNode* root, std::vector<LazyNode*>* interior) {
  if (root->op != LZ_MUL) return false;
  LazyNode* silu = node_of(root->in[0], LZ_MUL);
  if (!silu) return false;
  cg_tensor* g = silu->in[0];
  LazyNode* sig = node_of(silu->in[1], LZ_DIV);
  if (!sig || !scalar_is(sig->in[0], 1.0f)) return false;
  LazyNode* den = node_of(sig->in[1], LZ_ADD);
  if (!den || !scalar_is(den->in[0], 1.0f)) return false;
  LazyNode* ex = node_of(den->in[1], LZ_POW);
  if (!ex || !scalar_is(ex->in[0], 2.7182817f, 1e-6f)) return false;
  LazyNode* ng = node_of(ex->in[1], LZ_NEG);
  if (!ng || ng->in[0] != g || g->tag != CG_F32) return false;
  if (!same_shape(root->in[1], g)) return false;
  *interior = {ng, ex, den, sig, silu};
  root->m_t[0] = g;
  root->m_t[1] = root->in[1];
  root->m_i[0] = 0;
  return true;
}

// sigmoid(z) = div(one, add(one, pow(e, neg(z)))): returns z
cg_tensor* match_sigmoid(LazyNode* sig, std::vector<LazyNode*>* chain) {
  if (!sig || sig->op != LZ_DIV || !scalar_is(sig->in[0], 1.0f)) return nullptr;
  LazyNode* den = node_of(sig->in[1], LZ_ADD);
  if (!den || !scalar_is(den->in[0], 1.0f)) return nullptr;
  LazyNode* ex = node_of(den->in[1], LZ_POW);
  if (!ex || !scalar_is(ex->in[0], 2.7182817f, 1e-6f)) return nullptr;
  LazyNode* ng = node_of(ex->in[1], LZ_NEG);
  if (!ng) return nullptr;
  chain->push_back(ng);
  chain->push_back(ex);
  chain->push_back(den);
  chain->push_back(sig);
  return ng->in[0];
}

// gelu(g) * u with the tanh approximation spelled as nn/mod.rs:138-160 spells it:
// root = mul(mul(mul(0.5, g), add(1, sub(mul(2, sigmoid(mul(2, mul(c, add(g, mul(k, pow(g, 3))))))), 1))), u)
bool match_gelu_mul(LazyNode* root, std::vector<LazyNode*>* interior) {
  if (root->op != LZ_MUL) return false;
  LazyNode* gelu = node_of(root->in[0], LZ_MUL);
  if (!gelu) return false;
  LazyNode* hx = node_of(gelu->in[0], LZ_MUL);
  LazyNode* onep = node_of(gelu->in[1], LZ_ADD);
  if (!hx || !onep || !scalar_is(hx->in[0], 0.5f) || !scalar_is(onep->in[0], 1.0f)) return false;
  cg_tensor* g = hx->in[1];
  LazyNode* th = node_of(onep->in[1], LZ_SUB);
  if (!th || !scalar_is(th->in[1], 1.0f)) return false;
  LazyNode* two_s = node_of(th->in[0], LZ_MUL);
  if (!two_s || !scalar_is(two_s->in[0], 2.0f)) return false;
  std::vector<LazyNode*> chain;
  LazyNode* sig = node_of(two_s->in[1], LZ_DIV);
  cg_tensor* z = match_sigmoid(sig, &chain);
  LazyNode* zn = z ? node_of(z, LZ_MUL) : nullptr;
  if (!zn || !scalar_is(zn->in[0], 2.0f)) return false;
  LazyNode* y = node_of(zn->in[1], LZ_MUL);
  if (!y || !scalar_is(y->in[0], 0.7978845608f, 1e-6f)) return false;
  LazyNode* inner = node_of(y->in[1], LZ_ADD);
  if (!inner || inner->in[0] != g) return false;
  LazyNode* kx3 = node_of(inner->in[1], LZ_MUL);
  if (!kx3 || !scalar_is(kx3->in[0], 0.044715f, 1e-6f)) return false;
  LazyNode* x3 = node_of(kx3->in[1], LZ_POW);
  if (!x3 || x3->in[0] != g || !scalar_is(x3->in[1], 3.0f) || g->tag != CG_F32 || !same_shape(root->in[1], g)) return false;
  *interior = {x3, kx3, inner, y, zn};
  interior->insert(interior->end(), chain.begin(), chain.end());
  interior->push_back(two_s);
  interior->push_back(th);
  interior->push_back(onep);
  interior->push_back(hx);
  interior->push_back(gelu);
  root->m_t[0] = g;
  root->m_t[1] = root->in[1];
  root->m_i[0] = 1;
  return true;
}

// rope: root = add(mul(cos_b, x), mul(sin_b, concat(neg(slice(x, 3, d/2, d/2)), slice(x, 3, 0, d/2), 3)))
// with cos_b / sin_b concrete [.., S, d] views that only step over the last two axes
bool match_rope(LazyNode* root, std::vector<LazyNode*>* interior) {
  if (root->op != LZ_ADD) return false;
  LazyNode* mc = node_of(root->in[0], LZ_MUL);
  LazyNode* ms = node_of(root->in[1], LZ_MUL);
  if (!mc || !ms) return false;
  cg_tensor* x = mc->in[1];
  if (x->rank != 4 || x->tag != CG_F32 || x->strides[3] != 1 || (x->dims[3] & 1)) return false;
  const int64_t d = x->dims[3], half = d / 2;
  auto table = [&](const cg_tensor* t, int64_t* ld) -> const float* {
    if (!t || t->node || t->tag != CG_F32 || t->storage != ST_F32 || t->rank != 4 || !same_shape(t, x)) return nullptr;
    if ((t->dims[0] != 1 && t->strides[0] != 0) || (t->dims[1] != 1 && t->strides[1] != 0) || t->strides[3] != 1) return nullptr;
    *ld = t->strides[2];
    return (const float*)t->data();
  };
  int64_t ldc = 0, lds = 0;
  const float* ct = table(mc->in[0], &ldc);
  const float* st = table(ms->in[0], &lds);
  if (!ct || !st || ldc != lds) return false;
  LazyNode* rot = node_of(ms->in[1], LZ_CONCAT);
  if (!rot || rot->a[0] != 3) return false;
  LazyNode* ng = node_of(rot->in[0], LZ_NEG);
  if (!ng) return false;
  std::vector<LazyNode*> chain;
  if (!is_slice_of(ng->in[0], x, 3, half, half, &chain)) return false;
  if (!is_slice_of(rot->in[1], x, 3, 0, half, &chain)) return false;
  *interior = chain;
  interior->push_back(ng);
  interior->push_back(rot);
  interior->push_back(mc);
  interior->push_back(ms);
  root->m_t[0] = x;
  root->m_p[0] = ct;
  root->m_p[1] = st;
  root->m_i[0] = ldc;
  return true;
}

// repeat_kv: t = reshape(broadcast(reshape(base, [b, nkv, 1, S, d]), [b, nkv, rep, S, d]), [b, nkv * rep, S, d])
bool match_repeat(const cg_tensor* t, cg_tensor** base, int* rep, std::vector<LazyNode*>* chain) {
  LazyNode* r2 = producer(t);
  if (!r2 || r2->claimed || r2->fuse || (r2->op != LZ_RESHAPE_COPY && r2->op != LZ_RESHAPE) || t->rank != 4) return false;
  LazyNode* bc = node_of(r2->in[0], LZ_BROADCAST);
  if (!bc || bc->out->rank != 5) return false;
  LazyNode* r1 = node_of(bc->in[0], LZ_RESHAPE);
  if (!r1 || r1->out->rank != 5 || r1->out->dims[2] != 1) return false;
  cg_tensor* b0 = r1->in[0];
  if (b0->rank != 4) return false;
  const int64_t* d5 = bc->out->dims;
  if (d5[0] != b0->dims[0] || d5[1] != b0->dims[1] || d5[3] != b0->dims[2] || d5[4] != b0->dims[3]) return false;
  if (t->dims[0] != d5[0] || t->dims[1] != d5[1] * d5[2] || t->dims[2] != d5[3] || t->dims[3] != d5[4]) return false;
  *base = b0;
  *rep = (int)d5[2];
  chain->push_back(r1);
  chain->push_back(bc);
  chain->push_back(r2);
  return true;
}

// causal mask: t = broadcast(mul(cast(lt(row, col), F32), MIN)) with row = broadcast(reshape(arange(S), [S, 1]), [S, S])
// and col = broadcast(arange(S), [S, S])
bool match_causal_mask(const cg_tensor* t, int64_t S, std::vector<LazyNode*>* chain) {
  LazyNode* mb = node_of(t, LZ_BROADCAST);
  if (!mb) return false;
  LazyNode* mm = node_of(mb->in[0], LZ_MUL);
  if (!mm || !scalar_is(mm->in[1], -3.4028234663852886e38f)) return false;
  if (mm->out->rank != 2 || mm->out->dims[0] != S || mm->out->dims[1] != S) return false;
  LazyNode* cs = node_of(mm->in[0], LZ_CAST);
  if (!cs) return false;
  LazyNode* lt = node_of(cs->in[0], LZ_LT);
  if (!lt) return false;
  LazyNode* rowb = node_of(lt->in[0], LZ_BROADCAST);
  LazyNode* colb = node_of(lt->in[1], LZ_BROADCAST);
  if (!rowb || !colb) return false;
  LazyNode* rowr = node_of(rowb->in[0], LZ_RESHAPE);
  if (!rowr || rowr->out->rank != 2 || rowr->out->dims[0] != S || rowr->out->dims[1] != 1) return false;
  LazyNode* ar = node_of(rowr->in[0], LZ_ARANGE);
  LazyNode* ac = node_of(colb->in[0], LZ_ARANGE);
  if (!ar || !ac || ar->a[0] != S || ac->a[0] != S) return false;
  *chain = {ar, rowr, rowb, ac, colb, lt, cs, mm, mb};
  return true;
}

// attention core: root = matmul(softmax(add(div(matmul(q, transpose(k, 2, 3)), sqrt_d), mask_b)), v)
bool match_attention(LazyNode* root, std::vector<LazyNode*>* interior) {
  if (root->op != LZ_MATMUL || root->out->rank != 4) return false;
  LazyNode* pn = producer(root->in[0]);
  if (!pn || pn->claimed || pn->fuse) return false;
  std::vector<LazyNode*> sm;
  cg_tensor* scores = nullptr;
  if (!match_softmax(pn, &sm, &scores)) return false;
  LazyNode* plus = node_of(scores, LZ_ADD);
  if (!plus) return false;
  // the scale: div by a constant (llama.rs:100-102) or mul by one (granite.rs:155-156)
  LazyNode* scaled = producer(plus->in[0]);
  if (!scaled || scaled->claimed || scaled->fuse || (scaled->op != LZ_DIV && scaled->op != LZ_MUL)) return false;
  float scale;
  if (!scalar_f32(scaled->in[1], &scale)) return false;
  LazyNode* qk = node_of(scaled->in[0], LZ_MATMUL);
  if (!qk) return false;
  cg_tensor* q = qk->in[0];
  LazyNode* kt = node_of(qk->in[1], LZ_TRANSPOSE);
  if (!kt || !((kt->a[0] == 2 && kt->a[1] == 3) || (kt->a[0] == 3 && kt->a[1] == 2))) return false;
  cg_tensor* k = kt->in[0];
  cg_tensor* v = root->in[1];
  if (q->rank != 4 || k->rank != 4 || v->rank != 4 || q->tag != CG_F32) return false;
  const int64_t S = q->dims[2], d = q->dims[3];
  if (k->dims[2] != S || v->dims[2] != S || k->dims[3] != d || v->dims[3] != d) return false;  // prompt-shaped: no cache
  if (d != 64 && d != 128) return false;
  std::vector<LazyNode*> mask;
  if (!match_causal_mask(plus->in[1], S, &mask)) return false;
  // keys: rope(repeat(k0)) (llama / qwen3), repeat(k0') (gemma3: already rotated), or as given
  std::vector<LazyNode*> extra;
  cg_tensor *k0 = k, *v0 = v;
  int rep_k = 1, rep_v = 1;
  LazyNode* krope = nullptr;
  {
    std::vector<LazyNode*> rchain, pchain;
    LazyNode* kn = producer(k);
    cg_tensor* kb = nullptr;
    if (kn && !kn->claimed && !kn->fuse && match_rope(kn, &rchain) && match_repeat(kn->m_t[0], &kb, &rep_k, &pchain)) {
      krope = kn;
      k0 = kb;
      extra.insert(extra.end(), rchain.begin(), rchain.end());
      extra.insert(extra.end(), pchain.begin(), pchain.end());
      extra.push_back(kn);
    } else {
      rep_k = 1;
      pchain.clear();
      if (match_repeat(k, &kb, &rep_k, &pchain)) {
        k0 = kb;
        extra.insert(extra.end(), pchain.begin(), pchain.end());
      } else {
        rep_k = 1;
      }
    }
    std::vector<LazyNode*> vchain;
    cg_tensor* vb = nullptr;
    if (match_repeat(v, &vb, &rep_v, &vchain)) {
      v0 = vb;
      extra.insert(extra.end(), vchain.begin(), vchain.end());
    } else {
      rep_v = 1;
    }
  }
  if (rep_k != rep_v || k0->dims[1] != v0->dims[1] || k0->dims[1] * rep_k != q->dims[1] || k0->dims[0] != q->dims[0]) return false;
  if (k0->strides[3] != 1 || v0->strides[3] != 1 || q->strides[3] != 1) return false;
  *interior = sm;
  interior->push_back(pn);
  interior->push_back(plus);
  interior->push_back(scaled);
  interior->push_back(qk);
  interior->push_back(kt);
  interior->insert(interior->end(), mask.begin(), mask.end());
  interior->insert(interior->end(), extra.begin(), extra.end());
  root->m_t[0] = q;
  root->m_t[1] = k0;
  root->m_t[2] = v0;
  root->m_t[3] = krope ? krope->out : nullptr;  // marks "rotate k0 with krope's tables first"
  root->m_f = scale;
  root->m_i[0] = rep_k;
  root->m_i[1] = scaled->op == LZ_DIV ? 1 : 0;
  if (krope) {
    root->m_p[0] = krope->m_p[0];
    root->m_p[1] = krope->m_p[1];
    root->m_i[2] = krope->m_i[0];
  }
  return true;
}

// ------------------------------------------------------------------------------------------
// execution

int run_rope(cg_ctx* c, const cg_tensor* x, const float* ct, const float* st, int64_t ld, cg_tensor** out) {
  Hold xf;
  const cg_tensor* xs = x;
  if (x->storage != ST_F32) {
    CG_TRY(as_contiguous_f32(c, x, &xf.t));
    xs = xf.t;
  }
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, 4, &r.t));
  const int64_t n = r.t->numel() / 2;
  if (n) {
    k_rope_tab<<<grid_for(n, 256, 148 * 32), 256, 0, c->core->stream>>>((const float*)xs->data(), xs->strides[0], xs->strides[1],
                                                                      xs->strides[2], ct, st, ld, x->dims[1], x->dims[2], x->dims[3],
                                                                      n, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int run_attention(cg_ctx* c, LazyNode* root, cg_tensor** out) {
  cg_tensor *q = root->m_t[0], *k0 = root->m_t[1], *v0 = root->m_t[2];
  Hold kr;
  const cg_tensor* k = k0;
  if (root->m_t[3]) {  // rotate the un-repeated keys (rope commutes with repeat_kv: it acts per head and position)
    CG_TRY(run_rope(c, k0, root->m_p[0], root->m_p[1], root->m_i[2], &kr.t));
    k = kr.t;
  }
  const int rep = (int)root->m_i[0];
  const bool exact = c->precision == CG_PREC_F32 || !root->m_i[1];
  const int64_t S = q->dims[2], d = q->dims[3];
  if (!exact && !root->m_i[3]) {
    // bf16-precision context: the tensor-core attention (scores divided by sqrt(d) is what it computes)
    if (fabsf(root->m_f - sqrtf((float)d)) <= 1e-6f * root->m_f) return cg_fused_attention(c, q, k, v0, 0, 0.f, out);
  }
  if (q->storage != ST_F32 || k->storage != ST_F32 || v0->storage != ST_F32) return fail(c, CG_ERR_UNSUPPORTED, "lazy attention: f32 operands expected");
  const int out_bshd = (int)root->m_i[3];
  Hold r;
  if (out_bshd) CG_TRY(new_tensor(c, CG_F32, ST_F32, root->out->dims, root->out->rank, &r.t));  // [b, S, nh d]
  else CG_TRY(new_tensor(c, CG_F32, ST_F32, q->dims, 4, &r.t));
  // strides go to the kernel through a small device array (three axes each)
  int64_t hs[9] = {q->strides[0], q->strides[1], q->strides[2], k->strides[0], k->strides[1], k->strides[2],
                   v0->strides[0], v0->strides[1], v0->strides[2]};
  Hold sd;
  int64_t n18 = 18;
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n18, 1, &sd.t));
  CG_CUDA(c, cudaMemcpyAsync(sd.t->data(), hs, sizeof(hs), cudaMemcpyHostToDevice, c->core->stream));
  const int64_t* ds = (const int64_t*)sd.t->data();
  dim3 grid((unsigned)((S + 31) / 32), (unsigned)q->dims[1], (unsigned)q->dims[0]);
  if (grid.y > 65535 || grid.z > 65535) return fail(c, CG_ERR_UNSUPPORTED, "lazy attention: too many heads or rows");
  if (S) {
    const size_t smem = (size_t)(3 * 32 * (d + 1) + 32 * 33) * 4;
    static PerDeviceFlag big;
    if (d == 128 && !big.at(c->core->device)) {
      CG_CUDA(c, cudaFuncSetAttribute(k_attn_f32<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      big.at(c->core->device) = true;
    }
    if (d == 64)
      k_attn_f32<64><<<grid, 128, smem, c->core->stream>>>((const float*)q->data(), ds, (const float*)k->data(), ds + 3,
                                                        (const float*)v0->data(), ds + 6, S, rep, root->m_f, (int)root->m_i[1],
                                                        out_bshd, (float*)r.t->data());
    else
      k_attn_f32<128><<<grid, 128, smem, c->core->stream>>>((const float*)q->data(), ds, (const float*)k->data(), ds + 3,
                                                         (const float*)v0->data(), ds + 6, S, rep, root->m_f, (int)root->m_i[1],
                                                         out_bshd, (float*)r.t->data());
    CG_LAUNCHED(c);
  }
  *out = r.take();
  return CG_OK;
}

int run_fused(cg_ctx* c, LazyNode* n, cg_tensor** res) {
  switch (n->fuse) {
    case F_RMSNORM: {
      cg_tensor* x = n->m_t[0];
      Hold xc, r;
      CG_TRY(as_contiguous_f32(c, x, &xc.t));
      CG_TRY(new_tensor(c, CG_F32, ST_F32, x->dims, x->rank, &r.t));
      const int64_t H = x->dims[x->rank - 1], M = H ? x->numel() / H : 0;
      if (M && H) CG_TRY(k_launch_rmsnorm(c, (const float*)xc.t->data(), H, n->m_p[0], n->m_f, (int)n->m_i[0], M, H, r.t->data(), 0));
      *res = r.take();
      return CG_OK;
    }
    case F_SOFTMAX: return cg_fused_softmax(c, n->m_t[0], 0.f, res);
    case F_SILU_MUL: return cg_fused_act_mul(c, n->m_t[0], n->m_t[1], (int)n->m_i[0], res);
    case F_ROPE: return run_rope(c, n->m_t[0], n->m_p[0], n->m_p[1], n->m_i[0], res);
    case F_ATTENTION: return run_attention(c, n, res);
  }
  return fail(c, CG_ERR_INVALID, "lazy: unknown fused chain");
}

int run_node(cg_ctx* c, LazyNode* n) {
  cg_tensor* out = n->out;
  if (is_alias(n->op)) {
    // the metadata was computed when the view was recorded, relative to the (then already final)
    // layout of the input; only the storage has to be shared now
    out->buf = n->in[0]->buf;
    out->storage = n->in[0]->storage;
    out->node = nullptr;
    return CG_OK;
  }
  cg_tensor* res = nullptr;
  int st = CG_OK;
  if (n->fuse) {
    st = run_fused(c, n, &res);
    if (st == CG_OK) c->lazy_fused++;
  } else {
    cg_tensor *a = n->in[0], *b = n->in[1];
    switch (n->op) {
      case LZ_RESHAPE_COPY: {
        Hold cc;
        st = as_contiguous(c, a, &cc.t);
        if (st == CG_OK) st = cg_reshape(c, cc.t, n->a, n->na, &res);
        break;
      }
      case LZ_CAST: st = cg_cast(c, a, (int)n->a[0], &res); break;
      case LZ_ADD: st = cg_add(c, a, b, &res); break;
      case LZ_SUB: st = cg_sub(c, a, b, &res); break;
      case LZ_MUL: st = cg_mul(c, a, b, &res); break;
      case LZ_DIV: st = cg_div(c, a, b, &res); break;
      case LZ_POW: st = cg_pow(c, a, b, &res); break;
      case LZ_LT: st = cg_lt(c, a, b, &res); break;
      case LZ_NEG: st = cg_neg(c, a, &res); break;
      case LZ_MAX: st = cg_max(c, a, &res); break;
      case LZ_SUM: st = cg_sum(c, a, &res); break;
      case LZ_MATMUL: st = cg_matmul(c, a, b, &res); break;
      case LZ_CONCAT: st = cg_concat(c, a, b, (int)n->a[0], &res); break;
      case LZ_ARANGE: st = cg_arange(c, n->a[0], &res); break;
      default: st = fail(c, CG_ERR_INVALID, "lazy: unknown node");
    }
  }
  if (st != CG_OK) return st;
  if (!res->contiguous()) {
    cg_tensor* cc = nullptr;
    st = as_contiguous(c, res, &cc);
    release(res);
    if (st != CG_OK) return st;
    res = cc;
  }
  adopt(out, res);
  release(res);
  return CG_OK;
}

// Marks recognised chains.  Roots are tried from the last node backwards, so an attention core
// claims its softmax before the softmax is considered on its own.
void plan(cg_ctx* c) {
  std::vector<LazyNode*>& nodes = c->lazy_nodes;
  std::vector<std::vector<int>> readers(nodes.size());
  for (LazyNode* n : nodes) {
    if (n->dead) continue;
    for (int i = 0; i < n->nin; ++i)
      if (LazyNode* p = producer(n->in[i])) readers[p->index].push_back(n->index);
  }
  for (int i = (int)nodes.size() - 1; i >= 0; --i) {
    LazyNode* root = nodes[i];
    if (root->dead || root->claimed || root->fuse || is_alias(root->op)) continue;
    std::vector<LazyNode*> interior;
    int kind = F_NONE;
    cg_tensor* sx = nullptr;
    if (match_attention(root, &interior)) kind = F_ATTENTION;
    else if (interior.clear(), match_rmsnorm(root, &interior)) kind = F_RMSNORM;
    else if (interior.clear(), match_softmax(root, &interior, &sx)) { kind = F_SOFTMAX; root->m_t[0] = sx; }
    else if (interior.clear(), match_silu_mul(root, &interior)) kind = F_SILU_MUL;
    else if (interior.clear(), match_gelu_mul(root, &interior)) kind = F_SILU_MUL;
    else if (interior.clear(), match_rope(root, &interior)) kind = F_ROPE;
    if (!kind) continue;
    // every interior value must be private to the chain: read only inside it, no handle outside
    std::unordered_set<LazyNode*> inside(interior.begin(), interior.end());
    inside.insert(root);
    bool ok = true;
    for (LazyNode* m : interior) {
      if (m->claimed || m->fuse || m->dead || user_refs(m->out) > 0) { ok = false; break; }
      for (int r : readers[m->index])
        if (!inside.count(nodes[r])) { ok = false; break; }
      if (!ok) break;
    }
    if (!ok) continue;
    if (kind == F_ATTENTION && c->precision == CG_PREC_F32 && user_refs(root->out) == 0 && readers[root->index].size() == 1) {
      // llama.rs:110-112: the heads are put back beside each other by transpose(1, 2) + reshape, which
      // is a copy of the attention output; the f32 kernel can write that layout itself
      LazyNode* tr = nodes[readers[root->index][0]];
      if (tr->op == LZ_TRANSPOSE && !tr->claimed && !tr->fuse && !tr->dead && user_refs(tr->out) == 0 &&
          ((tr->a[0] == 1 && tr->a[1] == 2) || (tr->a[0] == 2 && tr->a[1] == 1)) && readers[tr->index].size() == 1) {
        LazyNode* cp = nodes[readers[tr->index][0]];
        const cg_tensor* q = root->m_t[0];
        if (cp->op == LZ_RESHAPE_COPY && !cp->claimed && !cp->fuse && !cp->dead && cp->out->rank == 3 && cp->out->dims[0] == q->dims[0] &&
            cp->out->dims[1] == q->dims[2] && cp->out->dims[2] == q->dims[1] * q->dims[3]) {
          for (int k = 0; k < 4; ++k) cp->m_t[k] = root->m_t[k];
          cp->m_p[0] = root->m_p[0]; cp->m_p[1] = root->m_p[1];
          cp->m_f = root->m_f;
          for (int k = 0; k < 3; ++k) cp->m_i[k] = root->m_i[k];
          cp->m_i[3] = 1;
          cp->fuse = F_ATTENTION;
          for (LazyNode* m : interior) m->claimed = cp;
          root->claimed = cp;
          tr->claimed = cp;
          continue;
        }
      }
    }
    root->fuse = kind;
    for (LazyNode* m : interior) m->claimed = root;
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// recorders

bool lazy_binary(cg_ctx* c, int op, const cg_tensor* a, const cg_tensor* b, cg_tensor** out, int* st) {
  if (a->tag != b->tag) { *st = fail(c, CG_ERR_DTYPE, "mixed dtypes in binary operation"); return true; }
  if (!same_shape(a, b)) { *st = fail(c, CG_ERR_SHAPE, "Shape mismatch in operation"); return true; }
  cg_tensor* t = pending_tensor(c, a->tag, a->dims, a->rank);
  static const int map[] = {LZ_ADD, LZ_SUB, LZ_MUL, LZ_DIV, LZ_POW, LZ_LT};
  add_node(c, map[op], t, a, b);
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_unary_neg(cg_ctx* c, const cg_tensor* x, cg_tensor** out, int* st) {
  cg_tensor* t = pending_tensor(c, x->tag, x->dims, x->rank);
  add_node(c, LZ_NEG, t, x, nullptr);
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_reduce(cg_ctx* c, int red, const cg_tensor* x, cg_tensor** out, int* st) {
  if (x->dims[x->rank - 1] >= (1ll << 32)) return false;  // the eager path reports it
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < x->rank; ++i) od[i] = x->dims[i];
  od[x->rank - 1] = 1;
  cg_tensor* t = pending_tensor(c, x->tag, od, x->rank);
  add_node(c, red == LR_MAX ? LZ_MAX : LZ_SUM, t, x, nullptr);
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_cast(cg_ctx* c, const cg_tensor* x, int dtype, cg_tensor** out, int* st) {
  if (!x->node && x->has_scalar) return false;  // a literal: cast it now so its value stays known
  cg_tensor* t = pending_tensor(c, dtype, x->dims, x->rank);
  LazyNode* n = add_node(c, LZ_CAST, t, x, nullptr);
  n->a[0] = dtype;
  n->na = 1;
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_matmul(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out, int* st) {
  const int ra = a->rank, rb = b->rank;
  if (a->tag != b->tag || ra < 2 || rb < 2 || ra != rb || a->dims[ra - 1] != b->dims[rb - 2]) return false;  // eager reports
  for (int i = 0; i < ra - 2; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < ra - 2; ++i) od[i] = a->dims[i];
  od[ra - 2] = a->dims[ra - 2];
  od[ra - 1] = b->dims[rb - 1];
  cg_tensor* t = pending_tensor(c, a->tag, od, ra);
  add_node(c, LZ_MATMUL, t, a, b);
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_concat(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, int dim, cg_tensor** out, int* st) {
  if (!a->node && !b->node) return false;  // nothing pending feeds it (the rotary tables): run it now
  if (a->tag != b->tag || a->rank != b->rank || dim < 0 || dim >= a->rank) return false;  // eager reports
  for (int i = 0; i < a->rank; ++i)
    if (i != dim && a->dims[i] != b->dims[i]) return false;
  int64_t od[CG_MAX_RANK];
  for (int i = 0; i < a->rank; ++i) od[i] = a->dims[i];
  od[dim] += b->dims[dim];
  cg_tensor* t = pending_tensor(c, a->tag, od, a->rank);
  LazyNode* n = add_node(c, LZ_CONCAT, t, a, b);
  n->a[0] = dim;
  n->na = 1;
  *out = t;
  *st = CG_OK;
  return true;
}

bool lazy_arange(cg_ctx* c, int64_t end, cg_tensor** out, int* st) {
  int64_t n1 = (int64_t)ceilf((float)end);
  cg_tensor* t = pending_tensor(c, CG_U32, &n1, 1);
  LazyNode* n = add_node(c, LZ_ARANGE, t, nullptr, nullptr);
  n->a[0] = end;
  n->na = 1;
  *out = t;
  *st = CG_OK;
  return true;
}

void lazy_view(cg_ctx* c, int kind, cg_tensor* t, const cg_tensor* x, const int64_t* args, int nargs) {
  LazyNode* n = add_node(c, kind, t, x, nullptr);
  n->na = std::min(nargs, CG_MAX_RANK + 2);
  for (int i = 0; i < n->na; ++i) n->a[i] = args[i];
}

int lazy_reshape_copy(cg_ctx* c, const cg_tensor* x, const int64_t* dims, int rank, cg_tensor** out) {
  cg_tensor* t = pending_tensor(c, x->tag, dims, rank);
  LazyNode* n = add_node(c, LZ_RESHAPE_COPY, t, x, nullptr);
  n->na = rank;
  for (int i = 0; i < rank; ++i) n->a[i] = dims[i];
  *out = t;
  return CG_OK;
}

void lazy_orphan(cg_tensor* t) {
  // the last handle to a value that was never computed is gone: nothing can read it any more
  // (readers hold references), so its node will not run
  LazyNode* n = t->node;
  t->node = nullptr;
  if (!n) return;
  n->dead = true;
  n->out = nullptr;
  drop_inputs(n);  // may orphan further nodes
}

int lazy_flush(cg_ctx* c) {
  if (!c || c->lazy_busy || c->lazy_nodes.empty()) return CG_OK;
  LazyPause busy(c);
  plan(c);
  std::vector<LazyNode*> nodes;
  nodes.swap(c->lazy_nodes);
  // a node lets go of its inputs once it has run; a node inside a chain once the chain's root has
  std::vector<std::vector<LazyNode*>> let_go(nodes.size());
  for (LazyNode* n : nodes) let_go[n->claimed ? n->claimed->index : n->index].push_back(n);
  int st = CG_OK;
  static const bool trace = getenv("CG_LAZY_TRACE") != nullptr;
  for (LazyNode* n : nodes) {
    if (!n->dead && !n->claimed && n->out) {
      const int64_t l0 = c->launches;
      if (st == CG_OK) st = run_node(c, n);
      if (trace && c->launches != l0)
        fprintf(stderr, "lazy: node %d op %d fuse %d -> %lld launches, out rank %d [%lld %lld %lld %lld]\n", n->index, n->op, n->fuse,
                (long long)(c->launches - l0), n->out ? n->out->rank : -1, n->out ? (long long)n->out->dims[0] : 0,
                n->out ? (long long)n->out->dims[1] : 0, n->out ? (long long)n->out->dims[2] : 0, n->out ? (long long)n->out->dims[3] : 0);
      if (st != CG_OK && n->out && n->out->buf == nullptr) {
        // leave no handle without contents behind: what could not be computed reads as zeros
        cg_tensor* z = nullptr;
        if (cg_zeros(c, n->out->dims, n->out->rank, n->out->tag, &z) == CG_OK) {
          adopt(n->out, z);
          release(z);
        } else {
          n->out->node = nullptr;
        }
      }
    }
    for (LazyNode* m : let_go[n->index]) {
      // (the value of a node inside a chain is never materialised; by the planner's check nothing
      // outside the chain can reach it, and it goes away with its last reader)
      if (m->out && m->out->node == m) m->out->node = nullptr;
      m->out = nullptr;
      drop_inputs(m);
    }
  }
  for (LazyNode* n : nodes) delete n;
  return st;
}

}  // namespace cg

using namespace cg;

extern "C" int32_t cg_lazy_stats(cg_ctx* c, int64_t* recorded, int64_t* fused, int64_t* pending) {
  if (!c) return CG_ERR_INVALID;
  if (recorded) *recorded = c->lazy_recorded;
  if (fused) *fused = c->lazy_fused;
  if (pending) *pending = (int64_t)c->lazy_nodes.size();
  return CG_OK;
}
