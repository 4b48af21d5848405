// decoder.cu — the greedy generation loop of catgrad-llm/examples/llama/main.rs:118-169 run
// natively on the device, for decoder-only models of the Llama family
// (catgrad-llm/src/models/llama.rs, with the switches of qwen3.rs / gemma3.rs).
//
// Where the reference recomputes the whole sequence for every generated token and passes
// pos = 0 (llama.rs:170-178), this runner keeps a device KV cache with the semantics of
// catgrad-llm/src/legacy/models/utils.rs:210-228 (append along the position axis), computes
// the LM head on the last position only, and feeds each step's argmax to the next step
// without a host round trip.  Position and token count live in device memory so that every
// decode step is the same kernel sequence: it is captured once into a CUDA graph and
// replayed.
//
// A decode step of a dense pre-norm layer is five kernels -- qkv GEMM, fused attention, o GEMM,
// paired gate/up GEMM, down GEMM -- with the RMSNorms folded into the GEMMs around them (see
// DecGemm in kernels.h); prefill runs the persistent tensor-core GEMMs and the tcgen05
// attention.  Mixture-of-experts layers (moe.cu) and post-norm models keep their norm kernels.
//
// Data layout in HBM (per rank; heads, FFN columns and vocabulary are sharded over tp_world):
//   w_qkv   [ (nh + 2 nkv) d, H ] bf16   rows = q heads, then k heads, then v heads
//   w_o     [ H, nh d ]           bf16
//   w_gu    [ 2 F, H ]            bf16   rows = gate, then up
//   w_down  [ H, F ]              bf16
//   experts [ E / W ][ Fe, H ] x2, [ E / W ][ H, Fe ] bf16 on mixture-of-experts layers (whole
//           experts per rank), router [ E, H ] f32
//   embed   [ V, H ]              bf16   (also the LM head when tied)
//   k/v     [ L ][ B, nkv, Tmax, d ] bf16
//   x       [ M, H ] f32 residual stream; bf16 only where a tensor-core GEMM reads it

#include <cstring>
#include <map>
#include <memory>
#include <string>

#include "kernels.h"
#include "nccl_dl.h"
#include "safetensors.h"

using namespace cg;

namespace {

struct Layer {
  cg_tensor *w_qkv = nullptr, *w_o = nullptr, *w_gu = nullptr, *w_down = nullptr;
  cg_tensor *ln_in = nullptr, *ln_post_attn = nullptr, *ln_pre_ffn = nullptr, *ln_post_ffn = nullptr;
  cg_tensor *q_norm = nullptr, *k_norm = nullptr;
  cg_tensor *k_cache = nullptr, *v_cache = nullptr;
  // mixture-of-experts layers (qwen3.rs:64-133): router [E, H] f32, this rank's experts stacked
  bool moe = false;
  cg_tensor *router = nullptr, *router3 = nullptr, *we_gate = nullptr, *we_up = nullptr, *we_down = nullptr;
};

void drop(cg_tensor*& t) {
  if (t) release(t);
  t = nullptr;
}

}  // namespace

struct cg_decoder {
  cg_ctx* c = nullptr;
  cg_decoder_config cfg{};
  std::map<std::string, cg_tensor*> params;  // as handed over, until finalize
  bool finalized = false;
  // sharded sizes
  int nh = 0, nkv = 0, d = 0, F = 0, Vp = 0, H = 0, qkv = 0;
  std::vector<Layer> layers;
  cg_tensor *embed = nullptr, *head = nullptr, *ln_f = nullptr;
  cg_tensor *cos_t = nullptr, *sin_t = nullptr;
  cg_tensor *cos_l = nullptr, *sin_l = nullptr;  // tables of the second rope base (gemma3.rs:154-159), or null
  // state
  cg_tensor* state = nullptr;     // int64[2] on device: {position, tokens generated}
  cg_tensor* cur = nullptr;       // u32 [B]: the tokens the next step consumes
  cg_tensor* history = nullptr;   // u32 [max_batch, max_seq]
  cg_tensor* logits = nullptr;    // f32 [tp_world, B, Vp]
  int64_t B = 0, pos = 0, generated = 0;
  // workspace (sized for `cap` tokens)
  int64_t cap = 0;
  cg_tensor *x = nullptr, *xn = nullptr, *qkvb = nullptr, *q = nullptr, *att = nullptr, *hact = nullptr,
            *tmp = nullptr, *xl = nullptr, *splitk = nullptr, *best = nullptr;
  // mixture-of-experts scratch, sized for cap * top_k pairs
  cg_tensor *m_ids = nullptr, *m_wts = nullptr, *m_pos = nullptr, *m_tiles = nullptr, *m_xg = nullptr, *m_h = nullptr,
            *m_y = nullptr, *m_xs3 = nullptr, *m_logits = nullptr;
  int El = 0;                    // experts on this rank
  int EW = 1, ER = 0;            // ranks the experts are split over, and this rank's place among them
  cg_tensor *ep_x = nullptr, *ep_y = nullptr;  // expert parallelism: every rank's rows gathered / this rank's expert sums for them
  bool pending_reduce = false;   // x still lacks the addends pushed by the last row-parallel GEMM
  // norm hand-over (see DecGemm): xn holds bf16(x * gain) un-normalised and ss the per-CTA sums
  // of squares the last residual GEMM wrote; the next GEMM applies 1 / rms in its epilogue
  bool xn_raw = false;
  bool xn_ready = false;         // xn already holds the normalised rows the next GEMM reads (post-norm models)
  int ss_parts = 0;
  cg_tensor* ss = nullptr;
  bool logits_gathered = true;   // `logits` holds every rank's slice
  cudaGraphExec_t graph = nullptr;
  int64_t graph_B = -1;
  int64_t graph_gen = -1;        // option generation the graph was captured under
  int64_t step_launches = 0;     // kernels in one decode step
  // all steps of a decode call as one resident kernel (decode_resident.cu), when the model allows
  ResidentPlan* rplan = nullptr;
  int64_t rplan_B = -1, rplan_gen = -1;
  bool resident_off = false;     // this model or device cannot take the resident kernel
  int64_t splitk_floats = 0;

  int64_t* pos_dev() { return (int64_t*)state->data(); }
  int64_t* count_dev() { return (int64_t*)state->data() + 1; }
};

namespace {

int all_reduce_f32(cg_decoder* D, float* p, int64_t n);
bool use_push(cg_decoder* D, int64_t M, int64_t S);

int get_param(cg_decoder* D, const std::string& name, cg_tensor** out, bool required = true) {
  auto it = D->params.find(name);
  if (it == D->params.end()) {
    *out = nullptr;
    return required ? fail(D->c, CG_ERR_INVALID, "decoder: missing parameter " + name) : CG_OK;
  }
  *out = it->second;
  return CG_OK;
}

// bf16 copy of rows [r0, r0 + nr) x cols [c0, c0 + nc) of a 2-D parameter, into dst at row `at`
int copy_block(cg_ctx* c, const cg_tensor* w, int64_t r0, int64_t nr, int64_t c0, int64_t nc, cg_tensor* dst, int64_t at) {
  if (w->rank != 2 || r0 + nr > w->dims[0] || c0 + nc > w->dims[1] || nc != dst->dims[1] || at + nr > dst->dims[0])
    return fail(c, CG_ERR_SHAPE, "decoder: parameter has an unexpected shape");
  cg_tensor *a = nullptr, *b = nullptr, *cv = nullptr;
  CG_TRY(cg_slice(c, w, 0, r0, nr, &a));
  Hold ha(a);
  CG_TRY(cg_slice(c, a, 1, c0, nc, &b));
  Hold hb(b);
  CG_TRY(cg_to_bf16(c, b, &cv));
  Hold hc(cv);
  CG_CUDA(c, cudaMemcpyAsync((char*)dst->data() + (size_t)at * nc * 2, cv->data(), (size_t)nr * nc * 2,
                             cudaMemcpyDeviceToDevice, c->core->stream));
  return CG_OK;
}

int norm_weight(cg_decoder* D, const std::string& name, int64_t n, cg_tensor** out, bool required = true) {
  cg_tensor* p = nullptr;
  CG_TRY(get_param(D, name, &p, required));
  if (!p) { *out = nullptr; return CG_OK; }
  if (p->numel() != n) return fail(D->c, CG_ERR_SHAPE, "decoder: " + name + " has an unexpected shape");
  return as_contiguous_f32(D->c, p, out);
}

int ensure_workspace(cg_decoder* D, int64_t M) {
  if (M <= D->cap) return CG_OK;
  cg_ctx* c = D->c;
  if (D->graph) { cudaGraphExecDestroy(D->graph); D->graph = nullptr; }  // it holds the old buffers
  if (D->rplan) { decode_resident_free(D->rplan); D->rplan = nullptr; D->rplan_B = -1; }
  drop(D->x); drop(D->xn); drop(D->qkvb); drop(D->q); drop(D->att); drop(D->hact); drop(D->tmp);
  const int64_t H = D->H;
  int64_t s2[2];
  s2[0] = M; s2[1] = H;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->x));
  s2[0] = M * (D->cfg.ep_world > 1 ? D->cfg.ep_world : 1);  // the expert block normalises every rank's rows
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->xn));
  s2[0] = M;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->tmp));
  s2[1] = D->qkv;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->qkvb));
  s2[1] = (int64_t)D->nh * D->d;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->q));
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->att));
  s2[1] = D->F;
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->hact));
  if (D->cfg.n_experts > 0) {
    drop(D->m_ids); drop(D->m_wts); drop(D->m_pos); drop(D->m_tiles); drop(D->m_xg); drop(D->m_h); drop(D->m_y);
    drop(D->m_xs3); drop(D->m_logits);
    const int64_t M_local = M;
    const int epw = D->cfg.ep_world > 1 ? D->cfg.ep_world : 1;
    M = M * epw;  // under expert parallelism the expert block sees the rows of every rank
    drop(D->ep_x); drop(D->ep_y);
    if (epw > 1) {
      s2[0] = M; s2[1] = H;
      CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->ep_x));
      CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->ep_y));
    }
    s2[0] = M; s2[1] = 3 * H;
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->m_xs3));
    s2[1] = D->cfg.n_experts;
    CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->m_logits));
    const int64_t P = M * D->cfg.top_k;
    int64_t n = P;
    CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->m_ids));
    CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &D->m_wts));
    CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->m_pos));
    n = 3 * P + 4;
    CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->m_tiles));
    s2[0] = P; s2[1] = H;
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->m_xg));
    CG_TRY(new_tensor(c, CG_F32, ST_F32, s2, 2, &D->m_y));
    s2[1] = D->cfg.moe_ffn;
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &D->m_h));
    // rows of a tile past its group are computed and discarded: keep them finite
    CG_CUDA(c, cudaMemsetAsync(D->m_xg->data(), 0, (size_t)P * H * 2, c->core->stream));
    CG_CUDA(c, cudaMemsetAsync(D->m_h->data(), 0, (size_t)P * D->cfg.moe_ffn * 2, c->core->stream));
    M = M_local;
  }
  D->cap = M;
  return CG_OK;
}

// x += t
__global__ void k_add_rows(float* x, const float* t, int64_t n) {
  const int64_t n4 = n / 4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 a = ((float4*)x)[i];
    const float4 b = ((const float4*)t)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    ((float4*)x)[i] = a;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) x[n4 * 4 + threadIdx.x] += t[n4 * 4 + threadIdx.x];
}

// The expert block of layer L on M tokens; under tensor parallelism every rank owns whole
// experts and the partial sums meet in the all-reduce of the residual stream.
int moe_block(cg_decoder* D, Layer& L, int64_t M, bool push = false) {
  const cg_decoder_config& cfg = D->cfg;
  const int64_t P = M * cfg.top_k;
  MoeArgs a;
  a.x = (const float*)D->x->data();
  a.out = (float*)D->x->data();
  a.gamma = (const float*)L.ln_pre_ffn->data();
  a.eps = cfg.rms_eps;
  a.plus_one = cfg.norm_plus_one;
  a.router = (const float*)L.router->data();
  a.router3 = (const __nv_bfloat16*)L.router3->data();
  a.xs3 = (__nv_bfloat16*)D->m_xs3->data();
  a.logits = (float*)D->m_logits->data();
  a.w_gate = (const __nv_bfloat16*)L.we_gate->data();
  a.w_up = (const __nv_bfloat16*)L.we_up->data();
  a.w_down = (const __nv_bfloat16*)L.we_down->data();
  a.H = (int)D->H; a.E = cfg.n_experts; a.k = cfg.top_k; a.Fe = cfg.moe_ffn; a.norm_topk = cfg.norm_topk; a.act = cfg.act;
  a.e_lo = D->ER * D->El; a.El = D->El;
  a.add_residual = cfg.tp_world > 1 && cfg.tp_rank != 0 ? 0 : 1;
  a.M = M;
  a.xn = (__nv_bfloat16*)D->xn->data();
  int32_t* t = (int32_t*)D->m_tiles->data();
  const int64_t Pc = D->cap * (cfg.ep_world > 1 ? cfg.ep_world : 1) * cfg.top_k;
  a.w.ids = (uint32_t*)D->m_ids->data();
  a.w.wts = (float*)D->m_wts->data();
  a.w.pos = (int32_t*)D->m_pos->data();
  a.w.tile_expert = t; a.w.tile_row0 = t + Pc; a.w.tile_rows = t + 2 * Pc; a.w.n_tiles = t + 3 * Pc;
  a.w.xg = (__nv_bfloat16*)D->m_xg->data();
  a.w.h = (__nv_bfloat16*)D->m_h->data();
  a.w.y = (float*)D->m_y->data();
  (void)P;
  if (cfg.ep_world > 1) {
    // Expert parallelism with data-parallel attention: gather every rank's rows, route them (the
    // same f32 arithmetic on the same numbers on every rank, so the expert ids agree everywhere),
    // run the experts this rank owns on all of them, and hand every rank the sum over all experts
    // for its own rows.
    cg_ctx* c = D->c;
    if (!c->comm) return fail(c, CG_ERR_COMM, "decoder: expert parallelism needs cg_comm_init first");
    const int64_t n = M * D->H;
    ncclResult_t r = nccl().AllGather(D->x->data(), D->ep_x->data(), (size_t)n, ncclFloat32, (ncclComm_t)c->comm, c->core->stream);
    if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllGather: ") + nccl().GetErrorString(r));
    a.x = (const float*)D->ep_x->data();
    a.out = (float*)D->ep_y->data();
    a.M = M * cfg.ep_world;
    a.add_residual = 0;
    CG_TRY(moe_ffn(c, a));
    r = nccl().ReduceScatter(D->ep_y->data(), D->tmp->data(), (size_t)n, ncclFloat32, ncclSum, (ncclComm_t)c->comm, c->core->stream);
    if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclReduceScatter: ") + nccl().GetErrorString(r));
    k_add_rows<<<grid_for((n + 3) / 4, 256), 256, 0, c->core->stream>>>((float*)D->x->data(), (const float*)D->tmp->data(), n);
    CG_LAUNCHED(c);
    return CG_OK;
  }
  PeerPush px;
  if (push) {
    // decode under tensor parallelism: no collective call (see project_add)
    px = peer_push_of(D->c->xchg);
    a.push = &px;
    return moe_ffn(D->c, a);
  }
  CG_TRY(moe_ffn(D->c, a));
  return all_reduce_f32(D, (float*)D->x->data(), M * D->H);
}

// y = x W^T (+ residual) on bf16 activations.  mode: 0 -> f32 out, 1 -> bf16 out,
// 2 -> out = residual + product (residual may alias out).  A handful of tokens takes the
// weight-streaming kernel (optionally with the fused gate/up epilogue), larger token counts
// the tiled kernel.
bool small_m(int64_t M, int64_t K) { return gemm_dec_supported(M, K); }

constexpr int SS_MAX_PARTS = 4096;

int gemm(cg_decoder* D, const cg_tensor* xin, int64_t M, const cg_tensor* w, void* out, const float* residual, int mode,
         bool dual = false, const cg_tensor* produce_gain = nullptr, bool consume = false) {
  const int64_t K = w->dims[1];
  const int64_t N = dual ? w->dims[0] / 2 : w->dims[0];
  if (small_m(M, K)) {
    DecGemm g;
    if (consume) {
      g.ss_in = (const float*)D->ss->data();
      g.ss_parts = D->ss_parts;
      g.ss_eps = D->cfg.rms_eps;
    }
    if (produce_gain) {
      g.xb_out = (__nv_bfloat16*)D->xn->data();
      g.g_next = (const float*)produce_gain->data();
      g.g_plus_one = D->cfg.norm_plus_one;
      g.ss_out = (float*)D->ss->data();
      D->ss_parts = gemm_dec_ss_parts(N, K);
      if (D->ss_parts > SS_MAX_PARTS) return fail(D->c, CG_ERR_UNSUPPORTED, "decoder: too many partial sums for the norm hand-over");
    }
    g.x = (const __nv_bfloat16*)xin->data(); g.ldx = K;
    g.w = (const __nv_bfloat16*)w->data(); g.ldw = K; g.w_rows = w->dims[0];
    g.out = out; g.ldo = N; g.residual = residual; g.out_mode = mode;
    PeerPush px;
    g.push = nullptr;
    if (mode == 3) { px = peer_push_of(D->c->xchg); g.push = &px; }
    g.dual = dual ? 1 : 0; g.act = D->cfg.act;
    g.M = M; g.N = N; g.K = K;
    return gemm_dec(D->c, g);
  }
  if (dual)
    return gemm_tc_pair(D->c, (const __nv_bfloat16*)xin->data(), K, (const __nv_bfloat16*)w->data(), K, (__nv_bfloat16*)out, N, M,
                        N, K, D->cfg.act);
  const int splits = gemm_tc_pick_splits(M, N, K);
  float* ws = (int64_t)splits * M * N <= D->splitk_floats ? (float*)D->splitk->data() : nullptr;
  return gemm_tc(D->c, (const __nv_bfloat16*)xin->data(), K, (const __nv_bfloat16*)w->data(), K, out, N, residual, M, N, K,
                 mode, splits, ws);
}

int all_reduce_f32(cg_decoder* D, float* p, int64_t n) {
  cg_ctx* c = D->c;
  if (D->cfg.tp_world <= 1) return CG_OK;
  if (!c->comm) return fail(c, CG_ERR_COMM, "decoder: tensor parallelism needs cg_comm_init first");
  ncclResult_t r = nccl().AllReduce(p, p, (size_t)n, ncclFloat32, ncclSum, (ncclComm_t)c->comm, c->core->stream);
  if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllReduce: ") + nccl().GetErrorString(r));
  return CG_OK;
}

int all_reduce_bf16(cg_decoder* D, __nv_bfloat16* p, int64_t n) {
  cg_ctx* c = D->c;
  if (D->cfg.tp_world <= 1) return CG_OK;
  if (!c->comm) return fail(c, CG_ERR_COMM, "decoder: tensor parallelism needs cg_comm_init first");
  ncclResult_t r = nccl().AllReduce(p, p, (size_t)n, ncclBfloat16, ncclSum, (ncclComm_t)c->comm, c->core->stream);
  if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllReduce: ") + nccl().GetErrorString(r));
  return CG_OK;
}

// x += W-projection of `xin` (row-split under tensor parallelism), optionally through a
// post-norm: x += rmsnorm(proj).
int project_add(cg_decoder* D, const cg_tensor* xin, int64_t M, const cg_tensor* w, const cg_tensor* post_norm, bool push,
                const cg_tensor* next_norm = nullptr) {
  cg_ctx* c = D->c;
  const bool tp = D->cfg.tp_world > 1;
  float* x = (float*)D->x->data();
  // decode under tensor parallelism: the GEMM pushes its partial product to every rank and
  // the norm that follows adds the partials of all ranks to x (no collective call)
  if (push) return gemm(D, xin, M, w, nullptr, nullptr, 3);
  if (!tp && !post_norm) return gemm(D, xin, M, w, x, x, 2);
  float* t = (float*)D->tmp->data();
  if (tp && !post_norm && !small_m(M, D->H) && D->H % 2 == 0 && D->cfg.n_experts == 0) {
    // prefill: the partial products travel as bf16 (half the bytes of the f32 residual stream;
    // the all-reduce is bandwidth-bound at these sizes), and one pass adds the reduced rows to
    // the replicated f32 residual and writes the norm the next block starts with.  Every rank
    // receives the same reduced rows, so the residual stream stays bit-identical across ranks.
    // Models with expert layers keep the f32 payload: a router sits behind the residual stream,
    // and a bf16-sized perturbation can flip a near-tie in its top-k, which the parity contract
    // (expert ids identical to the reference) does not allow.
    __nv_bfloat16* tb = (__nv_bfloat16*)D->tmp->data();
    CG_TRY(gemm(D, xin, M, w, tb, nullptr, 1));
    CG_TRY(all_reduce_bf16(D, tb, M * D->H));
    if (next_norm) D->xn_ready = true;
    return k_launch_add_bf16_norm(c, tb, next_norm ? (const float*)next_norm->data() : nullptr, D->cfg.rms_eps,
                                  D->cfg.norm_plus_one, M, D->H, x, (__nv_bfloat16*)D->xn->data());
  }
  if (tp && !post_norm) {
    // in place: rank 0 leaves x + partial in x, every other rank just its partial (its copy of
    // the old x is identical to rank 0's and no longer needed); the sum over ranks is the new
    // residual stream on every rank
    CG_TRY(gemm(D, xin, M, w, x, x, D->cfg.tp_rank == 0 ? 2 : 0));
    return all_reduce_f32(D, x, M * D->H);
  }
  CG_TRY(gemm(D, xin, M, w, t, nullptr, 0));
  CG_TRY(all_reduce_f32(D, t, M * D->H));
  if (next_norm) {
    // the norm the next block starts with, in the same pass: xn is ready afterwards
    D->xn_ready = true;
    return k_launch_rmsnorm_add_norm(c, t, (const float*)post_norm->data(), (const float*)next_norm->data(), D->cfg.rms_eps,
                                     D->cfg.norm_plus_one, M, D->H, x, (__nv_bfloat16*)D->xn->data());
  }
  return k_launch_rmsnorm_add(c, t, (const float*)post_norm->data(), D->cfg.rms_eps, D->cfg.norm_plus_one, M, D->H, x);
}

// The library-free reduction path serves decode steps of dense pre-norm models when the
// ranks could map each other's exchange areas.
bool use_push(cg_decoder* D, int64_t M, int64_t S) {
  const cg_decoder_config& cfg = D->cfg;
  return cfg.tp_world > 1 && D->c->xchg.ok && D->c->opt_peer && S == 1 && small_m(M, D->H) && !cfg.post_norms &&
         M * D->H <= D->c->xchg.max_elems;
}

// All layers for M = B * S new tokens at positions [pos0, pos0 + S); x holds the embeddings.
int run_layers(cg_decoder* D, int64_t B, int64_t S, int64_t pos0, bool from_dev_pos) {
  cg_ctx* c = D->c;
  const cg_decoder_config& cfg = D->cfg;
  const int64_t M = B * S;
  const bool push = use_push(D, M, S);
  const PeerPush px = push ? peer_push_of(c->xchg) : PeerPush{};
  D->pending_reduce = false;
  // norm hand-over between GEMMs: decode steps of pre-norm models on one GPU
  const bool handover = c->opt_handover && S == 1 && small_m(M, D->H) && cfg.tp_world == 1 && !cfg.post_norms;
  D->xn_raw = false;
  D->xn_ready = false;
  for (int li = 0; li < cfg.num_layers; ++li) {
    Layer& L = D->layers[li];
    const bool small = small_m(M, D->H);
    if (D->xn_raw || D->xn_ready) {
      // the previous layer's last kernel already left what the projection reads
    } else if (D->pending_reduce)
      CG_TRY(k_launch_rmsnorm_reduce(c, px, (float*)D->x->data(), D->H, (const float*)L.ln_in->data(), cfg.rms_eps,
                                     cfg.norm_plus_one, M, D->H, D->xn->data(), 1));
    else
      CG_TRY(k_launch_rmsnorm(c, (const float*)D->x->data(), D->H, (const float*)L.ln_in->data(), cfg.rms_eps,
                              cfg.norm_plus_one, M, D->H, D->xn->data(), 1));
    D->pending_reduce = false;
    D->xn_ready = false;
    CG_TRY(gemm(D, D->xn, M, L.w_qkv, D->qkvb->data(), nullptr, 0, false, nullptr, D->xn_raw));
    D->xn_raw = false;
    // layers off the pattern rotate with the local base (gemma3.rs:154-159)
    const bool local_rope = D->cos_l && cfg.rope_local_every > 0 && (li + 1) % cfg.rope_local_every != 0;
    const float* cos_t = (const float*)(local_rope ? D->cos_l : D->cos_t)->data();
    const float* sin_t = (const float*)(local_rope ? D->sin_l : D->sin_t)->data();
    const bool windowed = cfg.sliding_window > 0 && (cfg.window_every <= 1 || (li % cfg.window_every) != cfg.window_every - 1);
    if (S == 1) {
      AttnDecArgs f;
      f.push_merge = 0;  // (chosen by the launcher)
      f.qkv = (const float*)D->qkvb->data();
      f.cos_t = cos_t;
      f.sin_t = sin_t;
      f.q_gamma = L.q_norm ? (const float*)L.q_norm->data() : nullptr;
      f.k_gamma = L.k_norm ? (const float*)L.k_norm->data() : nullptr;
      f.norm_eps = cfg.rms_eps;
      f.norm_plus_one = cfg.norm_plus_one;
      f.k_cache = (__nv_bfloat16*)L.k_cache->data();
      f.v_cache = (__nv_bfloat16*)L.v_cache->data();
      f.out = (__nv_bfloat16*)D->att->data();
      f.pos_dev = from_dev_pos ? D->pos_dev() : nullptr;
      f.pos0 = pos0; f.Tmax = cfg.max_seq; f.B = B;
      f.nh = D->nh; f.nkv = D->nkv; f.d = D->d;
      f.window = windowed ? cfg.sliding_window : 0;
      f.softcap = cfg.attn_softcap;
      f.splits = attn_dec_splits(cfg.max_seq, B * D->nkv, D->d);
      CG_TRY(k_launch_attn_dec(c, f));
    } else {
    RopeStoreArgs r;
    r.qkv = (const float*)D->qkvb->data();
    r.cos_t = cos_t;
    r.sin_t = sin_t;
    r.q_gamma = L.q_norm ? (const float*)L.q_norm->data() : nullptr;
    r.k_gamma = L.k_norm ? (const float*)L.k_norm->data() : nullptr;
    r.norm_eps = cfg.rms_eps;
    r.norm_plus_one = cfg.norm_plus_one;
    r.q_out = (__nv_bfloat16*)D->q->data();
    r.k_cache = (__nv_bfloat16*)L.k_cache->data();
    r.v_cache = (__nv_bfloat16*)L.v_cache->data();
    r.M = M; r.S = S; r.pos0 = pos0; r.Tmax = cfg.max_seq;
    r.pos_dev = from_dev_pos ? D->pos_dev() : nullptr;
    r.nh = D->nh; r.nkv = D->nkv; r.d = D->d;
    CG_TRY(k_launch_rope_store(c, r));
    AttnArgs a;
    a.q = (const __nv_bfloat16*)D->q->data();
    a.k_cache = (const __nv_bfloat16*)L.k_cache->data();
    a.v_cache = (const __nv_bfloat16*)L.v_cache->data();
    a.out = (__nv_bfloat16*)D->att->data();
    a.B = B; a.S = S; a.pos0 = pos0; a.Tmax = cfg.max_seq;
    a.pos_dev = from_dev_pos ? D->pos_dev() : nullptr;
    a.nh = D->nh; a.nkv = D->nkv; a.d = D->d;
    a.window = windowed ? cfg.sliding_window : 0;
    a.softcap = cfg.attn_softcap;
    a.scratch = nullptr;
    CG_TRY(k_launch_attn_prefill(c, a));
    }
    if (!(handover && !L.moe))
      CG_TRY(project_add(D, D->att, M, L.w_o, L.ln_post_attn, push, cfg.post_norms && !L.moe ? L.ln_pre_ffn : nullptr));
    if (push && L.moe) {
      CG_TRY(moe_block(D, L, M, true));
      D->pending_reduce = true;
      continue;
    }
    if (push) {
      CG_TRY(k_launch_rmsnorm_reduce(c, px, (float*)D->x->data(), D->H, (const float*)L.ln_pre_ffn->data(), cfg.rms_eps,
                                     cfg.norm_plus_one, M, D->H, D->xn->data(), 1));
      CG_TRY(gemm(D, D->xn, M, L.w_gu, D->hact->data(), nullptr, 1, true));
      CG_TRY(project_add(D, D->hact, M, L.w_down, nullptr, true));
      D->pending_reduce = true;
      continue;
    }
    if (handover && !L.moe) {
      float* x = (float*)D->x->data();
      CG_TRY(gemm(D, D->att, M, L.w_o, x, x, 2, false, L.ln_pre_ffn));
      CG_TRY(gemm(D, D->xn, M, L.w_gu, D->hact->data(), nullptr, 1, true, nullptr, true));
      const cg_tensor* next_gain = li + 1 < cfg.num_layers ? D->layers[li + 1].ln_in : D->ln_f;
      CG_TRY(gemm(D, D->hact, M, L.w_down, x, x, 2, false, next_gain));
      D->xn_raw = true;
      continue;
    }
    if (L.moe) {
      CG_TRY(moe_block(D, L, M));
      continue;
    }
    if (!D->xn_ready)
      CG_TRY(k_launch_rmsnorm(c, (const float*)D->x->data(), D->H, (const float*)L.ln_pre_ffn->data(), cfg.rms_eps,
                              cfg.norm_plus_one, M, D->H, D->xn->data(), 1));
    D->xn_ready = false;
    // gate/up projections and act(gate) * up in one kernel
    CG_TRY(gemm(D, D->xn, M, L.w_gu, D->hact->data(), nullptr, 1, true));
    (void)small;
    CG_TRY(project_add(D, D->hact, M, L.w_down, L.ln_post_ffn, false,
                       cfg.post_norms && li + 1 < cfg.num_layers ? D->layers[li + 1].ln_in : nullptr));
  }
  return CG_OK;
}

// Final norm on the last position of every row, LM head, greedy pick.
int run_head(cg_decoder* D, int64_t B, int64_t S, bool advance) {
  cg_ctx* c = D->c;
  const cg_decoder_config& cfg = D->cfg;
  float* lg = (float*)D->logits->data();
  float* mine = lg + (int64_t)cfg.tp_rank * B * D->Vp;
  if (D->xn_raw) {
    // decode step with the norm hand-over (S == 1): the LM head reads bf16(x * gain) and scales
    D->xn_raw = false;
    CG_TRY(gemm(D, D->xn, B, D->head, mine, nullptr, 0, false, nullptr, true));
    D->logits_gathered = true;
    return k_launch_argmax(c, lg, B, D->Vp, cfg.tp_world, cfg.final_softcap, (uint32_t*)D->cur->data(),
                           (uint32_t*)D->history->data(), cfg.max_seq, D->count_dev(), D->pos_dev(), advance ? 1 : 0,
                           (unsigned long long*)D->best->data());
  }
  if (D->pending_reduce) {
    // decode step on the push path: S == 1
    const PeerPush px = peer_push_of(c->xchg);
    CG_TRY(k_launch_rmsnorm_reduce(c, px, (float*)D->x->data(), D->H, (const float*)D->ln_f->data(), cfg.rms_eps,
                                   cfg.norm_plus_one, B, D->H, D->xl->data(), 1));
    D->pending_reduce = false;
    CG_TRY(gemm(D, D->xl, B, D->head, mine, nullptr, 0));
    D->logits_gathered = false;
    return k_launch_argmax_tp(c, px, mine, B, D->Vp, cfg.final_softcap, (uint32_t*)D->cur->data(),
                              (uint32_t*)D->history->data(), cfg.max_seq, D->count_dev(), D->pos_dev(), advance ? 1 : 0,
                              (unsigned long long*)D->best->data());
  }
  CG_TRY(k_launch_rmsnorm(c, (const float*)D->x->data() + (S - 1) * D->H, S * D->H, (const float*)D->ln_f->data(),
                          cfg.rms_eps, cfg.norm_plus_one, B, D->H, D->xl->data(), 1));
  CG_TRY(gemm(D, D->xl, B, D->head, mine, nullptr, 0));
  D->logits_gathered = true;
  if (cfg.tp_world > 1) {
    if (!c->comm) return fail(c, CG_ERR_COMM, "decoder: tensor parallelism needs cg_comm_init first");
    ncclResult_t r = nccl().AllGather(mine, lg, (size_t)(B * D->Vp), ncclFloat32, (ncclComm_t)c->comm, c->core->stream);
    if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllGather: ") + nccl().GetErrorString(r));
  }
  return k_launch_argmax(c, lg, B, D->Vp, cfg.tp_world, cfg.final_softcap, (uint32_t*)D->cur->data(),
                         (uint32_t*)D->history->data(), cfg.max_seq, D->count_dev(), D->pos_dev(), advance ? 1 : 0,
                         (unsigned long long*)D->best->data());
}

// One decode step for B rows reading position / count from device memory.
int enqueue_step(cg_decoder* D, int64_t B) {
  cg_ctx* c = D->c;
  CG_TRY(k_launch_embed(c, (const uint32_t*)D->cur->data(), 1, 0, 1, D->embed->data(), D->embed->storage, D->cfg.vocab, B,
                        D->H, D->cfg.embed_scale > 0.f ? D->cfg.embed_scale : 1.f, (float*)D->x->data()));
  CG_TRY(run_layers(D, B, 1, 0, true));
  return run_head(D, B, 1, true);
}

int logits_copy(cg_decoder* D, cg_tensor** out) {
  if (!out) return CG_OK;
  cg_ctx* c = D->c;
  const int W = D->cfg.tp_world;
  if (W > 1 && !D->logits_gathered) {
    // the push path leaves every rank with its own vocabulary slice only
    float* lg = (float*)D->logits->data();
    ncclResult_t r = nccl().AllGather(lg + (int64_t)D->cfg.tp_rank * D->B * D->Vp, lg, (size_t)(D->B * D->Vp), ncclFloat32,
                                      (ncclComm_t)c->comm, c->core->stream);
    if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllGather: ") + nccl().GetErrorString(r));
    D->logits_gathered = true;
  }
  int64_t od[2] = {D->B, (int64_t)D->Vp * W};
  Hold r;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, od, 2, &r.t));
  // [W, B, Vp] -> [B, W * Vp]
  for (int w = 0; w < W; ++w)
    CG_CUDA(c, cudaMemcpy2DAsync((float*)r.t->data() + (int64_t)w * D->Vp, (size_t)od[1] * 4,
                                 (const float*)D->logits->data() + (int64_t)w * D->B * D->Vp, (size_t)D->Vp * 4,
                                 (size_t)D->Vp * 4, (size_t)D->B, cudaMemcpyDeviceToDevice, c->core->stream));
  *out = r.take();
  return CG_OK;
}

// The resident decode kernel serves dense pre-norm models on one GPU (Llama, dense Qwen3).
bool resident_model(cg_decoder* D, ResidentModel* m) {
  const cg_decoder_config& cfg = D->cfg;
  if (cfg.tp_world != 1 || cfg.post_norms) return false;
  for (const Layer& L : D->layers)
    if (L.moe) return false;
  m->layers.resize(D->layers.size());
  for (size_t li = 0; li < D->layers.size(); ++li) {
    const Layer& L = D->layers[li];
    ResidentLayerDesc& d = m->layers[li];
    d.w_qkv = (const __nv_bfloat16*)L.w_qkv->data(); d.w_o = (const __nv_bfloat16*)L.w_o->data();
    d.w_gu = (const __nv_bfloat16*)L.w_gu->data(); d.w_down = (const __nv_bfloat16*)L.w_down->data();
    d.gain_in = (const float*)L.ln_in->data(); d.gain_ffn = (const float*)L.ln_pre_ffn->data();
    d.q_gamma = L.q_norm ? (const float*)L.q_norm->data() : nullptr;
    d.k_gamma = L.k_norm ? (const float*)L.k_norm->data() : nullptr;
    const bool local_rope = D->cos_l && cfg.rope_local_every > 0 && ((int)li + 1) % cfg.rope_local_every != 0;
    d.cos_t = (const float*)(local_rope ? D->cos_l : D->cos_t)->data();
    d.sin_t = (const float*)(local_rope ? D->sin_l : D->sin_t)->data();
    d.k_cache = (__nv_bfloat16*)L.k_cache->data(); d.v_cache = (__nv_bfloat16*)L.v_cache->data();
    const bool windowed = cfg.sliding_window > 0 && (cfg.window_every <= 1 || ((int)li % cfg.window_every) != cfg.window_every - 1);
    d.window = windowed ? cfg.sliding_window : 0;
  }
  m->head = (const __nv_bfloat16*)D->head->data();
  m->gain_final = (const float*)D->ln_f->data();
  m->embed = D->embed->data();
  m->embed_storage = D->embed->storage;
  m->H = D->H; m->F = D->F; m->Vp = D->Vp; m->vocab = cfg.vocab; m->Tmax = cfg.max_seq;
  m->nh = D->nh; m->nkv = D->nkv; m->d = D->d; m->act = cfg.act; m->plus_one = cfg.norm_plus_one;
  m->eps = cfg.rms_eps; m->attn_softcap = cfg.attn_softcap; m->final_softcap = cfg.final_softcap;
  m->embed_scale = cfg.embed_scale > 0.f ? cfg.embed_scale : 1.f;
  m->x = (float*)D->x->data(); m->xn = (__nv_bfloat16*)D->xn->data();
  m->ss = (float*)D->ss->data(); m->ss_parts_cap = SS_MAX_PARTS;
  m->qkv = (float*)D->qkvb->data(); m->att = (__nv_bfloat16*)D->att->data(); m->hact = (__nv_bfloat16*)D->hact->data();
  m->logits = (float*)D->logits->data();
  m->cur = (uint32_t*)D->cur->data(); m->history = (uint32_t*)D->history->data(); m->hist_ld = cfg.max_seq;
  m->count_dev = D->count_dev(); m->pos_dev = D->pos_dev();
  m->best = (unsigned long long*)D->best->data();
  return true;
}

// Runs `steps` decode steps on the resident kernel when the model and the context allow it.
// *ran says whether it did.
int try_resident(cg_decoder* D, int steps, bool* ran) {
  *ran = false;
  cg_ctx* c = D->c;
  if (!c->opt_resident || D->resident_off) return CG_OK;
  if (!D->rplan || D->rplan_B != D->B || D->rplan_gen != c->opt_generation) {
    if (D->rplan) { decode_resident_free(D->rplan); D->rplan = nullptr; D->rplan_B = -1; }
    ResidentModel m;
    if (!resident_model(D, &m) || !decode_resident_supported(m, D->B)) { D->resident_off = true; return CG_OK; }
    int st = decode_resident_prepare(c, m, D->B, &D->rplan);
    if (st == CG_ERR_UNSUPPORTED) { D->resident_off = true; c->err.clear(); return CG_OK; }
    CG_TRY(st);
    D->rplan_B = D->B;
    D->rplan_gen = c->opt_generation;
  }
  CG_TRY(decode_resident_run(c, D->rplan, steps));
  D->logits_gathered = true;
  *ran = true;
  return CG_OK;
}

__global__ void k_set_state(int64_t* state, int64_t pos, int64_t generated) {
  state[0] = pos;
  state[1] = generated;
}

// The device copy of {position, tokens generated}, set in stream order by a one-thread kernel:
// no host buffer is involved, so nothing has to be waited for.
int set_state(cg_decoder* D, int64_t pos, int64_t generated) {
  k_set_state<<<1, 1, 0, D->c->core->stream>>>((int64_t*)D->state->data(), pos, generated);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(D->c, e, "k_set_state");
  D->c->launches++;
  D->pos = pos;
  D->generated = generated;
  return CG_OK;
}

}  // namespace

extern "C" {

int32_t cg_decoder_create(cg_ctx* c, const cg_decoder_config* cfg, cg_decoder** out) {
  if (!c || !cfg || !out) return fail(c, CG_ERR_INVALID, "null argument");
  const cg_decoder_config& k = *cfg;
  if (k.num_layers <= 0 || k.hidden <= 0 || k.n_heads <= 0 || k.n_kv_heads <= 0 || k.head_dim <= 0 || k.ffn <= 0 ||
      k.vocab <= 0 || k.max_seq <= 0 || k.max_batch <= 0)
    return fail(c, CG_ERR_INVALID, "decoder: sizes must be positive");
  const int W = k.tp_world < 1 ? 1 : k.tp_world;
  if (k.n_experts > 0) {
    if (k.top_k < 1 || k.top_k > 32 || k.top_k > k.n_experts || k.moe_ffn <= 0 || k.moe_ffn % 8 || k.n_experts % W)
      return fail(c, CG_ERR_UNSUPPORTED,
                  "decoder: experts per token must be in [1, 32], the expert width a multiple of 8, experts divisible by the "
                  "parallel degree");
    if (k.post_norms) return fail(c, CG_ERR_UNSUPPORTED, "decoder: expert layers with post-norms are not supported");
  }
  if (k.tp_rank < 0 || k.tp_rank >= W) return fail(c, CG_ERR_INVALID, "decoder: tp_rank out of range");
  const int EPW = k.ep_world < 1 ? 1 : k.ep_world;
  if (EPW > 1 && (W != 1 || k.n_experts <= 0 || k.n_experts % EPW || k.ep_rank < 0 || k.ep_rank >= EPW))
    return fail(c, CG_ERR_INVALID, "decoder: expert parallelism needs tp_world = 1, experts divisible by ep_world and ep_rank in range");
  // fewer kv heads than ranks: every kv head is replicated on W / n_kv_heads consecutive ranks
  const bool kv_ok = k.n_kv_heads % W == 0 || (k.n_kv_heads < W && W % k.n_kv_heads == 0);
  if (k.n_heads % k.n_kv_heads || k.n_heads % W || !kv_ok || k.ffn % W || k.vocab % W)
    return fail(c, CG_ERR_SHAPE, "decoder: heads, kv heads, ffn and vocab must divide by the tensor-parallel degree");
  if (k.hidden % 8 || (k.ffn / W) % 8 || (k.vocab / W) % 8 || k.head_dim % 8)
    return fail(c, CG_ERR_UNSUPPORTED, "decoder: hidden, ffn, vocab shards and head_dim must be multiples of 8");
  if (c->precision != CG_PREC_BF16) return fail(c, CG_ERR_UNSUPPORTED, "decoder: needs a bf16-precision context");
  auto* D = new cg_decoder();
  D->c = c;
  D->cfg = k;
  D->cfg.tp_world = W;
  D->H = k.hidden;
  D->nh = k.n_heads / W;
  D->nkv = k.n_kv_heads >= W ? k.n_kv_heads / W : 1;
  D->d = k.head_dim;
  D->F = k.ffn / W;
  D->Vp = k.vocab / W;
  D->qkv = (D->nh + 2 * D->nkv) * D->d;
  D->EW = EPW > 1 ? EPW : W;
  D->ER = EPW > 1 ? k.ep_rank : k.tp_rank;
  D->El = k.n_experts > 0 ? k.n_experts / D->EW : 0;
  *out = D;
  return CG_OK;
}

int32_t cg_decoder_destroy(cg_decoder* D) {
  if (!D) return CG_ERR_INVALID;
  cudaStreamSynchronize(D->c->core->stream);
  if (D->graph) cudaGraphExecDestroy(D->graph);
  if (D->rplan) decode_resident_free(D->rplan);
  for (auto& kv : D->params) release(kv.second);
  for (auto& L : D->layers) {
    drop(L.w_qkv); drop(L.w_o); drop(L.w_gu); drop(L.w_down); drop(L.ln_in); drop(L.ln_post_attn);
    if (L.ln_pre_ffn) drop(L.ln_pre_ffn);
    drop(L.ln_post_ffn); drop(L.q_norm); drop(L.k_norm); drop(L.k_cache); drop(L.v_cache);
    drop(L.router); drop(L.router3); drop(L.we_gate); drop(L.we_up); drop(L.we_down);
  }
  if (D->head != D->embed) drop(D->head);
  drop(D->embed); drop(D->ln_f); drop(D->cos_t); drop(D->sin_t); drop(D->cos_l); drop(D->sin_l); drop(D->state); drop(D->cur); drop(D->history);
  drop(D->logits); drop(D->x); drop(D->xn); drop(D->qkvb); drop(D->q); drop(D->att); drop(D->hact);
  drop(D->tmp); drop(D->xl); drop(D->splitk); drop(D->best); drop(D->ss);
  drop(D->m_ids); drop(D->m_wts); drop(D->m_pos); drop(D->m_tiles); drop(D->m_xg); drop(D->m_h); drop(D->m_y);
  drop(D->m_xs3); drop(D->m_logits); drop(D->ep_x); drop(D->ep_y);
  delete D;
  return CG_OK;
}

int32_t cg_decoder_set_param(cg_decoder* D, const char* name, const cg_tensor* t) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !name || !t) return CG_ERR_INVALID;
  if (D->finalized) return fail(D->c, CG_ERR_INVALID, "decoder: already finalized");
  const_cast<cg_tensor*>(t)->rc++;
  auto it = D->params.find(name);
  if (it != D->params.end()) { release(it->second); it->second = const_cast<cg_tensor*>(t); }
  else D->params.emplace(name, const_cast<cg_tensor*>(t));
  return CG_OK;
}

// Checkpoint file -> decoder parameters (catgrad-llm/examples/llama/main.rs:279-354 and the
// expert stacking of :173-264).  Every tensor crosses the host link once, in the element type the
// file stores (bf16 stays bf16).  Per-expert matrices "...mlp.experts.{e}.{proj}.weight" land
// directly in slot e of the stacked "[E, rows, cols]" tensor the expert block reads, allocated
// when the layer's first expert shows up: one pass, where the reference concatenates the experts
// pairwise (quadratic copying).  Several files (shards) may be loaded one after another.
int32_t cg_decoder_load_safetensors(cg_decoder* D, const char* path) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !path) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (D->finalized) return fail(c, CG_ERR_INVALID, "decoder: already finalized");
  std::string why;
  std::unique_ptr<cg_safetensors> f(st_open(path, &why));
  if (!f) return fail(c, CG_ERR_INVALID, "safetensors: " + why);
  for (const StEntry& e : f->entries) {
    int layer = -1, expert = -1, used = 0;
    char proj[32] = {0};
    if (sscanf(e.name.c_str(), "model.layers.%d.mlp.experts.%d.%31[a-z_].weight%n", &layer, &expert, proj, &used) == 3 &&
        used == (int)e.name.size()) {
      if (e.dims.size() != 2 || expert < 0 || expert >= D->cfg.n_experts)
        return fail(c, CG_ERR_SHAPE, "decoder: " + e.name + " is not a matrix of one of the configured experts");
      const std::string stacked = "model.layers." + std::to_string(layer) + ".mlp.experts." + proj + ".weight";
      auto it = D->params.find(stacked);
      if (it == D->params.end()) {
        int64_t d3[3] = {D->cfg.n_experts, e.dims[0], e.dims[1]};
        cg_tensor* t = nullptr;
        CG_TRY(new_tensor(c, CG_F32, ST_BF16, d3, 3, &t));
        it = D->params.emplace(stacked, t).first;
      }
      cg_tensor* dst = it->second;
      if (dst->rank != 3 || dst->dims[1] != e.dims[0] || dst->dims[2] != e.dims[1])
        return fail(c, CG_ERR_SHAPE, "decoder: the experts of " + stacked + " differ in shape");
      CG_TRY(st_upload_into_bf16(c, f.get(), e, dst, (int64_t)expert * e.dims[0] * e.dims[1]));
      continue;
    }
    cg_tensor* t = nullptr;
    CG_TRY(st_upload(c, f.get(), e, &t));
    Hold h(t);
    CG_TRY(cg_decoder_set_param(D, e.name.c_str(), t));
  }
  // the copies read the mapping, which goes away with `f`
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  return CG_OK;
}

int32_t cg_decoder_finalize(cg_decoder* D) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (D->finalized) return CG_OK;
  const cg_decoder_config& cfg = D->cfg;
  const int W = cfg.tp_world, R = cfg.tp_rank;
  const int64_t H = D->H, d = D->d;
  const int64_t nh_all = cfg.n_heads, nkv_all = cfg.n_kv_heads;
  D->layers.resize(cfg.num_layers);
  for (int li = 0; li < cfg.num_layers; ++li) {
    Layer& L = D->layers[li];
    const std::string p = "model.layers." + std::to_string(li) + ".";
    cg_tensor *wq, *wk, *wv, *wo, *wg = nullptr, *wu = nullptr, *wd = nullptr, *wr = nullptr;
    CG_TRY(get_param(D, p + "self_attn.q_proj.weight", &wq));
    CG_TRY(get_param(D, p + "self_attn.k_proj.weight", &wk));
    CG_TRY(get_param(D, p + "self_attn.v_proj.weight", &wv));
    CG_TRY(get_param(D, p + "self_attn.o_proj.weight", &wo));
    // a layer is sparse when the checkpoint has a router for it (qwen3.rs:297-298)
    if (cfg.n_experts > 0) CG_TRY(get_param(D, p + "mlp.gate.weight", &wr, false));
    L.moe = wr != nullptr;
    if (L.moe) {
      const int64_t E = cfg.n_experts, Fe = cfg.moe_ffn, El = D->El;
      cg_tensor *eg, *eu, *ed;
      CG_TRY(get_param(D, p + "mlp.experts.gate_proj.weight", &eg));
      CG_TRY(get_param(D, p + "mlp.experts.up_proj.weight", &eu));
      CG_TRY(get_param(D, p + "mlp.experts.down_proj.weight", &ed));
      if (wr->rank != 2 || wr->dims[0] != E || wr->dims[1] != H || eg->rank != 3 || eg->dims[0] != E || eg->dims[1] != Fe ||
          eg->dims[2] != H || eu->rank != 3 || eu->dims[0] != E || eu->dims[1] != Fe || eu->dims[2] != H || ed->rank != 3 ||
          ed->dims[0] != E || ed->dims[1] != H || ed->dims[2] != Fe)
        return fail(c, CG_ERR_SHAPE, "decoder: expert parameters have unexpected shapes");
      CG_TRY(as_contiguous_f32(c, wr, &L.router));
      {
        // the router matrix three times along k, for the split-precision router GEMM
        Hold rb;
        CG_TRY(cg_to_bf16(c, wr, &rb.t));
        int64_t r3[2] = {E, 3 * H};
        CG_TRY(new_tensor(c, CG_F32, ST_BF16, r3, 2, &L.router3));
        for (int rep3 = 0; rep3 < 3; ++rep3)
          CG_CUDA(c, cudaMemcpy2DAsync((__nv_bfloat16*)L.router3->data() + rep3 * H, (size_t)3 * H * 2, rb.t->data(), (size_t)H * 2,
                                       (size_t)H * 2, (size_t)E, cudaMemcpyDeviceToDevice, c->core->stream));
        CG_CUDA(c, cudaStreamSynchronize(c->core->stream));  // rb is released at the end of this scope
      }
      for (auto pr : {std::make_pair(eg, &L.we_gate), std::make_pair(eu, &L.we_up), std::make_pair(ed, &L.we_down)}) {
        cg_tensor* sl = nullptr;
        CG_TRY(cg_slice(c, pr.first, 0, (int64_t)D->ER * El, El, &sl));
        Hold hs(sl);
        if (sl->storage == ST_BF16 && sl->contiguous()) { sl->rc++; *pr.second = sl; }  // already in the layout the GEMM reads
        else CG_TRY(cg_to_bf16(c, sl, pr.second));
      }
      for (const char* n : {"mlp.gate.weight", "mlp.experts.gate_proj.weight", "mlp.experts.up_proj.weight",
                            "mlp.experts.down_proj.weight"}) {
        auto it = D->params.find(p + n);
        if (it != D->params.end()) { release(it->second); D->params.erase(it); }
      }
    } else {
      CG_TRY(get_param(D, p + "mlp.gate_proj.weight", &wg));
      CG_TRY(get_param(D, p + "mlp.up_proj.weight", &wu));
      CG_TRY(get_param(D, p + "mlp.down_proj.weight", &wd));
    }
    if (wq->rank != 2 || wq->dims[0] != nh_all * d || wk->rank != 2 || wk->dims[0] != nkv_all * d || wv->rank != 2 ||
        wv->dims[0] != nkv_all * d)
      return fail(c, CG_ERR_SHAPE, "decoder: attention projections have unexpected shapes");
    int64_t s2[2] = {D->qkv, H};
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &L.w_qkv));
    CG_TRY(copy_block(c, wq, (int64_t)R * D->nh * d, D->nh * d, 0, H, L.w_qkv, 0));
    // this rank's kv heads: its own share, or the one head its query heads belong to
    const int64_t kv0 = nkv_all >= W ? (int64_t)R * D->nkv : (int64_t)R * nkv_all / W;
    CG_TRY(copy_block(c, wk, kv0 * d, D->nkv * d, 0, H, L.w_qkv, D->nh * d));
    CG_TRY(copy_block(c, wv, kv0 * d, D->nkv * d, 0, H, L.w_qkv, (D->nh + D->nkv) * d));
    s2[0] = H; s2[1] = D->nh * d;
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &L.w_o));
    CG_TRY(copy_block(c, wo, 0, H, (int64_t)R * D->nh * d, D->nh * d, L.w_o, 0));
    if (!L.moe) {
      s2[0] = 2 * (int64_t)D->F; s2[1] = H;
      CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &L.w_gu));
      CG_TRY(copy_block(c, wg, (int64_t)R * D->F, D->F, 0, H, L.w_gu, 0));
      CG_TRY(copy_block(c, wu, (int64_t)R * D->F, D->F, 0, H, L.w_gu, D->F));
      s2[0] = H; s2[1] = D->F;
      CG_TRY(new_tensor(c, CG_F32, ST_BF16, s2, 2, &L.w_down));
      CG_TRY(copy_block(c, wd, 0, H, (int64_t)R * D->F, D->F, L.w_down, 0));
    }
    CG_TRY(norm_weight(D, p + "input_layernorm.weight", H, &L.ln_in));
    if (cfg.post_norms) {
      // four norms per layer (catgrad-llm/src/models/gemma3.rs:192-238)
      CG_TRY(norm_weight(D, p + "post_attention_layernorm.weight", H, &L.ln_post_attn));
      CG_TRY(norm_weight(D, p + "pre_feedforward_layernorm.weight", H, &L.ln_pre_ffn));
      CG_TRY(norm_weight(D, p + "post_feedforward_layernorm.weight", H, &L.ln_post_ffn));
    } else {
      CG_TRY(norm_weight(D, p + "post_attention_layernorm.weight", H, &L.ln_pre_ffn));
    }
    if (cfg.qk_norm) {
      CG_TRY(norm_weight(D, p + "self_attn.q_norm.weight", d, &L.q_norm));
      CG_TRY(norm_weight(D, p + "self_attn.k_norm.weight", d, &L.k_norm));
    }
    int64_t s4[4] = {cfg.max_batch, D->nkv, cfg.max_seq, d};
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s4, 4, &L.k_cache));
    CG_TRY(new_tensor(c, CG_F32, ST_BF16, s4, 4, &L.v_cache));
    CG_CUDA(c, cudaMemsetAsync(L.k_cache->data(), 0, (size_t)L.k_cache->numel() * 2, c->core->stream));
    CG_CUDA(c, cudaMemsetAsync(L.v_cache->data(), 0, (size_t)L.v_cache->numel() * 2, c->core->stream));
    // the originals of this layer are no longer needed
    for (const char* n : {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                          "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"}) {
      auto it = D->params.find(p + n);
      if (it != D->params.end()) { release(it->second); D->params.erase(it); }
    }
  }
  {
    cg_tensor* e = nullptr;
    CG_TRY(get_param(D, "model.embed_tokens.weight", &e));
    if (e->rank != 2 || e->dims[0] != cfg.vocab || e->dims[1] != H) return fail(c, CG_ERR_SHAPE, "decoder: embedding shape");
    if (e->storage == ST_BF16 && e->contiguous()) { e->rc++; D->embed = e; }
    else CG_TRY(cg_to_bf16(c, e, &D->embed));
    cg_tensor* hsrc = D->embed;
    Hold htmp;
    if (!cfg.tie_embeddings) {
      cg_tensor* h = nullptr;
      CG_TRY(get_param(D, "lm_head.weight", &h));
      if (h->rank != 2 || h->dims[0] != cfg.vocab || h->dims[1] != H) return fail(c, CG_ERR_SHAPE, "decoder: lm_head shape");
      if (h->storage == ST_BF16 && h->contiguous()) { h->rc++; htmp.t = h; }
      else CG_TRY(cg_to_bf16(c, h, &htmp.t));
      hsrc = htmp.t;
    }
    // this rank's vocabulary slice is a row range of the table: a view, no copy
    cg_tensor* hv = nullptr;
    CG_TRY(cg_slice(c, hsrc, 0, (int64_t)R * D->Vp, D->Vp, &hv));
    D->head = hv;
    CG_TRY(norm_weight(D, "model.norm.weight", H, &D->ln_f));
  }
  for (auto& kv : D->params) release(kv.second);
  D->params.clear();
  (void)W;

  int64_t td[2] = {cfg.max_seq, d / 2};
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &D->cos_t));
  CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &D->sin_t));
  RopeScaling rs;
  rs.kind = cfg.rope_scaling; rs.factor = cfg.rope_factor; rs.low_freq_factor = cfg.rope_low_freq_factor;
  rs.high_freq_factor = cfg.rope_high_freq_factor; rs.beta_fast = cfg.rope_beta_fast; rs.beta_slow = cfg.rope_beta_slow;
  rs.original_max_pos = cfg.rope_original_max_pos;
  CG_TRY(k_launch_rope_tables_scaled(c, cfg.rope_theta, rs, cfg.max_seq, d, (float*)D->cos_t->data(), (float*)D->sin_t->data()));
  if (cfg.rope_local_theta > 0.f && cfg.rope_local_every > 0) {
    CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &D->cos_l));
    CG_TRY(new_tensor(c, CG_F32, ST_F32, td, 2, &D->sin_l));
    CG_TRY(k_launch_rope_tables(c, cfg.rope_local_theta, cfg.max_seq, d, (float*)D->cos_l->data(), (float*)D->sin_l->data()));
  }

  int64_t n = 4;
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->state));  // 16 bytes: two int64
  n = cfg.max_batch;
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->cur));
  int64_t hd[2] = {cfg.max_batch, cfg.max_seq};
  CG_TRY(new_tensor(c, CG_U32, ST_U32, hd, 2, &D->history));
  int64_t ld[3] = {cfg.tp_world, cfg.max_batch, D->Vp};
  CG_TRY(new_tensor(c, CG_F32, ST_F32, ld, 3, &D->logits));
  int64_t xd[2] = {cfg.max_batch, H};
  CG_TRY(new_tensor(c, CG_F32, ST_BF16, xd, 2, &D->xl));
  // split-K partials: at most 32 slices of a [tokens <= 64, widest GEMM output] problem
  const int64_t widest = std::max<int64_t>(std::max<int64_t>(D->qkv, 2 * (int64_t)D->F), std::max<int64_t>(H, D->Vp));
  n = std::max<int64_t>(32 * 64 * widest, (int64_t)300 * 128 * 256);
  CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &D->splitk));
  D->splitk_floats = n;
  n = (int64_t)SS_MAX_PARTS * 32;
  CG_TRY(new_tensor(c, CG_F32, ST_F32, &n, 1, &D->ss));
  n = 2 * (int64_t)cfg.max_batch;  // one 64-bit argmax merge slot per row
  CG_TRY(new_tensor(c, CG_U32, ST_U32, &n, 1, &D->best));
  CG_CUDA(c, cudaMemsetAsync(D->best->data(), 0, (size_t)n * 4, c->core->stream));

  CG_TRY(ensure_workspace(D, cfg.max_batch));
  CG_TRY(set_state(D, 0, 0));
  D->finalized = true;
  return cg_sync(c);
}

int32_t cg_decoder_reset(cg_decoder* D) {
  if (!D || !D->finalized) return CG_ERR_INVALID;
  D->B = 0;
  return set_state(D, 0, 0);
}

}  // extern "C"

namespace {

// Runs `tokens` [B, S] through the model at cache positions [base, base + S), appends their keys
// and values, and leaves the greedy next token of every row in the token buffer (counted as
// generated token number `generated`).
int prefill_at(cg_decoder* D, const cg_tensor* tokens, int64_t base, int64_t generated, cg_tensor** logits_out) {
  cg_ctx* c = D->c;
  if (tokens->tag != CG_U32 || tokens->rank != 2) return fail(c, CG_ERR_SHAPE, "decoder: tokens must be U32 [B, S]");
  const int64_t B = tokens->dims[0], S = tokens->dims[1];
  if (B < 1 || B > D->cfg.max_batch || S < 1 || base + S > D->cfg.max_seq) return fail(c, CG_ERR_SHAPE, "decoder: batch or length out of range");
  if (generated >= D->cfg.max_seq) return fail(c, CG_ERR_SHAPE, "decoder: token history is full");
  Hold tk;
  CG_TRY(as_contiguous(c, tokens, &tk.t));
  CG_TRY(set_state(D, base, generated));
  D->B = B;
  // the prompt is processed in position chunks so the workspace stays bounded
  const int64_t chunk_tokens = c->opt_prefill_chunk;
  int64_t Sc = std::max<int64_t>(1, chunk_tokens / B);
  if (Sc > 64) Sc = Sc / 64 * 64;
  Sc = std::min(Sc, S);
  CG_TRY(ensure_workspace(D, B * Sc));
  for (int64_t p0 = 0; p0 < S; p0 += Sc) {
    const int64_t s = std::min(Sc, S - p0);
    CG_TRY(k_launch_embed(c, (const uint32_t*)tk.t->data(), S, p0, s, D->embed->data(), D->embed->storage, D->cfg.vocab,
                          B * s, D->H, D->cfg.embed_scale > 0.f ? D->cfg.embed_scale : 1.f, (float*)D->x->data()));
    // a one-token chunk would take the decode attention path, which reads the device position
    if (s == 1) CG_TRY(set_state(D, base + p0, generated));
    CG_TRY(run_layers(D, B, s, base + p0, s == 1));
    if (p0 + s == S) {
      CG_TRY(set_state(D, base + S, generated));
      CG_TRY(run_head(D, B, s, false));
      // count the new token (the position stays base + S: that token is not cached yet)
      CG_TRY(set_state(D, base + S, generated + 1));
    }
  }
  return logits_copy(D, logits_out);
}

}  // namespace

extern "C" {

int32_t cg_decoder_prefill(cg_decoder* D, const cg_tensor* tokens, cg_tensor** logits_out) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !tokens) return CG_ERR_INVALID;
  if (!D->finalized) return fail(D->c, CG_ERR_INVALID, "decoder: finalize first");
  return prefill_at(D, tokens, 0, 0, logits_out);
}

int32_t cg_decoder_append(cg_decoder* D, const cg_tensor* tokens, cg_tensor** logits_out) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !tokens) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (!D->finalized) return fail(c, CG_ERR_INVALID, "decoder: finalize first");
  if (D->B == 0) return prefill_at(D, tokens, 0, 0, logits_out);  // nothing cached yet
  if (tokens->rank != 2 || tokens->dims[0] != D->B) return fail(c, CG_ERR_SHAPE, "decoder: append needs the cached batch size");
  return prefill_at(D, tokens, D->pos, D->generated, logits_out);
}

int32_t cg_decoder_truncate(cg_decoder* D, int64_t positions) {
  if (!D || !D->finalized) return CG_ERR_INVALID;
  if (positions < 0 || positions > D->pos) return fail(D->c, CG_ERR_INVALID, "decoder: cannot truncate to more positions than are cached");
  if (positions == 0) D->B = 0;
  return set_state(D, positions, 0);
}

int32_t cg_decoder_position(cg_decoder* D, int64_t* cached, int64_t* generated) {
  if (!D) return CG_ERR_INVALID;
  if (cached) *cached = D->pos;
  if (generated) *generated = D->generated;
  return CG_OK;
}

int32_t cg_decoder_decode(cg_decoder* D, int32_t steps, cg_tensor** logits_out) {
  if (!D || steps < 0) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (!D->finalized || D->B == 0) return fail(c, CG_ERR_INVALID, "decoder: prefill first");
  if (D->pos + steps > D->cfg.max_seq) return fail(c, CG_ERR_SHAPE, "decoder: KV cache capacity exceeded");
  if (steps == 0) return logits_copy(D, logits_out);
  {
    bool ran = false;
    CG_TRY(try_resident(D, steps, &ran));
    if (ran) {
      D->pos += steps;
      D->generated += steps;
      return logits_copy(D, logits_out);
    }
  }
  cudaStream_t s = c->core->stream;
  if (!D->graph || D->graph_B != D->B || D->graph_gen != c->opt_generation) {
    if (D->graph) { cudaGraphExecDestroy(D->graph); D->graph = nullptr; }
    // Run one step eagerly first: it configures kernel attributes and surfaces errors
    // outside of capture.  Then capture the identical sequence.
    const int64_t before = c->launches;
    CG_TRY(enqueue_step(D, D->B));
    D->step_launches = c->launches - before;
    D->pos += 1;
    D->generated += 1;
    steps -= 1;
    cudaGraph_t g = nullptr;
    CG_CUDA(c, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int st = enqueue_step(D, D->B);
    cudaError_t e = cudaStreamEndCapture(s, &g);
    c->launches = before + D->step_launches;  // capturing launched nothing
    if (st != CG_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) return cuda_fail(c, e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&D->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(c, e, "cudaGraphInstantiate");
    D->graph_B = D->B;
    D->graph_gen = c->opt_generation;
  }
  for (int i = 0; i < steps; ++i) CG_CUDA(c, cudaGraphLaunch(D->graph, s));
  c->launches += (int64_t)steps * D->step_launches;  // each replay runs the captured kernels
  D->pos += steps;
  D->generated += steps;
  return logits_copy(D, logits_out);
}

int32_t cg_decoder_step_with(cg_decoder* D, const cg_tensor* tokens, cg_tensor** logits_out) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !tokens) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (!D->finalized || D->B == 0) return fail(c, CG_ERR_INVALID, "decoder: prefill first");
  if (tokens->tag != CG_U32 || tokens->numel() != D->B) return fail(c, CG_ERR_SHAPE, "decoder: tokens must be U32 [B]");
  if (D->pos + 1 > D->cfg.max_seq) return fail(c, CG_ERR_SHAPE, "decoder: KV cache capacity exceeded");
  Hold tk;
  CG_TRY(as_contiguous(c, tokens, &tk.t));
  CG_CUDA(c, cudaMemcpyAsync(D->cur->data(), tk.t->data(), (size_t)D->B * 4, cudaMemcpyDeviceToDevice, c->core->stream));
  bool ran = false;
  CG_TRY(try_resident(D, 1, &ran));
  if (!ran) CG_TRY(enqueue_step(D, D->B));
  D->pos += 1;
  D->generated += 1;
  return logits_copy(D, logits_out);
}

int32_t cg_decoder_time_gemms(cg_decoder* D, int32_t batch, int32_t iters, float* ms_per_sweep, int32_t* launches_per_sweep) {
  if (!D || !ms_per_sweep || iters < 1) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (!D->finalized) return fail(c, CG_ERR_INVALID, "decoder: finalize first");
  if (batch < 1 || batch > D->cfg.max_batch) return fail(c, CG_ERR_SHAPE, "decoder: batch out of range");
  const int64_t M = batch;
  CG_TRY(ensure_workspace(D, M));
  cudaEvent_t e0, e1;
  CG_CUDA(c, cudaEventCreate(&e0));
  CG_CUDA(c, cudaEventCreate(&e1));
  int st = CG_OK;
  int64_t before = 0;
  for (int it = -1; it < iters && st == CG_OK; ++it) {  // iteration -1 warms up
    if (it == 0) { cudaEventRecord(e0, c->core->stream); before = c->launches; }
    const bool small = small_m(M, D->H);
    for (int li = 0; li < D->cfg.num_layers && st == CG_OK; ++li) {
      Layer& L = D->layers[li];
      st = gemm(D, D->xn, M, L.w_qkv, D->qkvb->data(), nullptr, 0);
      if (st == CG_OK) st = gemm(D, D->att, M, L.w_o, D->tmp->data(), nullptr, 0);
      if (L.moe) continue;  // the expert GEMMs depend on the routing: not part of this sweep
      if (st == CG_OK) st = gemm(D, D->xn, M, L.w_gu, D->hact->data(), nullptr, 1, true);
      (void)small;
      if (st == CG_OK) st = gemm(D, D->hact, M, L.w_down, D->tmp->data(), nullptr, 0);
    }
    if (st == CG_OK) st = gemm(D, D->xl, M, D->head, D->logits->data(), nullptr, 0);
  }
  cudaEventRecord(e1, c->core->stream);
  cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (st != CG_OK) return st;
  *ms_per_sweep = ms / (float)iters;
  if (launches_per_sweep) *launches_per_sweep = (int32_t)((c->launches - before) / iters);
  return cg_sync(c);
}

int32_t cg_decoder_resident_trace(cg_decoder* D, int32_t cta, uint64_t* out, int32_t n) {
  if (!D) return CG_ERR_INVALID;
  if (!D->rplan) return fail(D->c, CG_ERR_INVALID, "decoder: the resident kernel has not run yet");
  return decode_resident_trace(D->c, D->rplan, cta, out, n);
}

int32_t cg_decoder_tokens(cg_decoder* D, cg_tensor** out) {
  if (!D || !out) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  if (!D->finalized) return fail(c, CG_ERR_INVALID, "decoder: finalize first");
  cg_tensor *a = nullptr, *b = nullptr;
  CG_TRY(cg_slice(c, D->history, 0, 0, D->B, &a));
  Hold ha(a);
  CG_TRY(cg_slice(c, a, 1, 0, D->generated, &b));
  Hold hb(b);
  return as_contiguous(c, b, out);
}

int32_t cg_decoder_generate(cg_decoder* D, const uint32_t* prompt, int32_t batch, int32_t seq, int32_t n_decode,
                            uint32_t* out) {
  CG_LAZY_EAGER_SCOPE(D ? D->c : nullptr);
  if (!D || !prompt || !out || batch < 1 || seq < 1 || n_decode < 0) return CG_ERR_INVALID;
  cg_ctx* c = D->c;
  cg_tensor* tk = nullptr;
  int64_t dims[2] = {batch, seq};
  CG_TRY(cg_ndarray_from_vec_u32(c, prompt, (int64_t)batch * seq, dims, 2, &tk));
  Hold htk(tk);
  CG_TRY(cg_decoder_prefill(D, tk, nullptr));
  CG_TRY(cg_decoder_decode(D, n_decode, nullptr));
  // The reference reads every step's token back before the next forward (main.rs:160) because
  // its host loop feeds it in again; here the device feeds itself, so all steps are enqueued
  // back to back and the token history [batch, 1 + n_decode] comes back in one strided copy.
  const int64_t ld = 1 + (int64_t)n_decode;
  CG_CUDA(c, cudaMemcpy2DAsync(out, (size_t)ld * 4, D->history->data(), (size_t)D->cfg.max_seq * 4, (size_t)ld * 4, (size_t)batch,
                               cudaMemcpyDeviceToHost, c->core->stream));
  return cg_sync(c);
}

}  // extern "C"
