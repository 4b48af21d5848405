// kernels.h — launchers of the fused kernels shared by the public fused entry points and
// the decoder runner.  All pointers are device pointers; all arrays are contiguous
// row-major unless a leading dimension is given.
#pragma once

#include <vector>

#include "runtime.h"

namespace cg {

// x[m, :] = table[tok(m), :] * scale (table f32 or bf16), where row m = b * S + s reads
// tokens[b * tok_ld + tok_off + s]: a window of S positions out of a [B, tok_ld] id matrix.
int k_launch_embed(cg_ctx* c, const uint32_t* tokens, int64_t tok_ld, int64_t tok_off, int64_t S, const void* table,
                   int table_storage, int64_t vocab, int64_t M, int64_t H, float scale, float* out);

// RMSNorm of each row of x [M, H] (row stride ldx): out = x / sqrt(mean(x^2) + eps) * g, g = gamma or 1 + gamma.
// out_bf16 selects the output element type (bf16 feeds the tensor-core GEMMs).
int k_launch_rmsnorm(cg_ctx* c, const float* x, int64_t ldx, const float* gamma, float eps, int plus_one, int64_t M,
                     int64_t H, void* out, int out_bf16);
// In-place residual update with a normalised addend: x += rmsnorm(y) (post-norm layers).
int k_launch_rmsnorm_add(cg_ctx* c, const float* y, const float* gamma, float eps, int plus_one, int64_t M, int64_t H,
                         float* x);

// x += rmsnorm(y; g1) and, in the same pass, out = bf16(rmsnorm(x; g2)): a post-norm followed by
// the next block's pre-norm.
int k_launch_rmsnorm_add_norm(cg_ctx* c, const float* y, const float* g1, const float* g2, float eps, int plus_one, int64_t M,
                              int64_t H, float* x, __nv_bfloat16* out);

// x += t (bf16 rows into the f32 residual stream) and, when g is non-null, out = bf16(rmsnorm(x; g))
// in the same pass: the tail of a tensor-parallel row-parallel projection after its bf16 all-reduce.
int k_launch_add_bf16_norm(cg_ctx* c, const __nv_bfloat16* t, const float* g, float eps, int plus_one, int64_t M, int64_t H,
                           float* x, __nv_bfloat16* out);

// act(gu[m, 0:F]) * gu[m, F:2F] -> bf16 [M, F]; act 0 = silu, 1 = tanh-gelu.
int k_launch_act_mul(cg_ctx* c, const float* gu, int64_t M, int64_t F, int act, __nv_bfloat16* out);

// Rotary tables exactly as the reference builds them: cos/sin [T, d/2] f32.
int k_launch_rope_tables(cg_ctx* c, float theta, int64_t T, int64_t d, float* cos_t, float* sin_t);
// The same with the frequency rescaling of long-context checkpoints
// (catgrad-llm/src/legacy/nn/rope.rs:32-201): kind 1 = "llama3" (low frequencies divided by
// `factor`, a smooth blend between the two wavelength thresholds), kind 2 = "yarn" (linear ramp
// between interpolated and extrapolated frequencies, tables scaled by 0.1 ln(factor) + 1).
struct RopeScaling {
  int kind = 0;  // 0 none, 1 llama3, 2 yarn
  float factor = 1.f, low_freq_factor = 1.f, high_freq_factor = 4.f, beta_fast = 32.f, beta_slow = 1.f;
  int original_max_pos = 0;
};
int k_launch_rope_tables_scaled(cg_ctx* c, float theta, const RopeScaling& rs, int64_t T, int64_t d, float* cos_t, float* sin_t);

struct RopeStoreArgs {
  const float* qkv;        // [M, (nh + 2 nkv) d]
  const float* cos_t;      // [T, d/2]
  const float* sin_t;
  const float* q_gamma;    // optional per-head norm weights [d] (null = none)
  const float* k_gamma;
  float norm_eps;
  int norm_plus_one;
  __nv_bfloat16* q_out;    // [M, nh d]
  __nv_bfloat16* k_cache;  // [B, nkv, Tmax, d]
  __nv_bfloat16* v_cache;
  int64_t M, S;            // M = B * S tokens; token m is row m / S at position pos0 + m % S
  int64_t pos0, Tmax;
  const int64_t* pos_dev;  // when non-null, pos0 is read from device memory instead
  int nh, nkv, d;
};
// Split qkv, optionally normalise q/k per head, rotate q and k, write q (bf16) and append k, v
// to the cache.
int k_launch_rope_store(cg_ctx* c, const RopeStoreArgs& a);

struct AttnArgs {
  const __nv_bfloat16* q;        // [B * S, nh d]
  const __nv_bfloat16* k_cache;  // [B, nkv, Tmax, d]
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [B * S, nh d]
  int64_t B, S, pos0, Tmax;
  const int64_t* pos_dev;        // decode only: when non-null, pos0 is read from device memory
  int nh, nkv, d;
  int64_t window;                // 0 = none
  float softcap;                 // 0 = none
  float* scratch;                // unused
};
// Causal (optionally windowed / soft-capped) attention of S new tokens per row against cache
// positions [0, pos0 + S).  Tensor-core flash kernel.
int k_launch_attn_prefill(cg_ctx* c, const AttnArgs& a);

// The same on tcgen05 / TMEM for head sizes 64 and 128 without soft-cap or window (attention_fa.cu);
// k_launch_attn_prefill routes here by itself when the context allows it.
bool attn_fa_supported(const AttnArgs& a);
int k_launch_attn_fa(cg_ctx* c, const AttnArgs& a);

struct AttnDecArgs {
  const float* qkv;              // [B, (nh + 2 nkv) d] f32: the fused projection of the new tokens
  const float* cos_t;            // rotary tables [Tmax, d/2]
  const float* sin_t;
  const float* q_gamma;          // optional per-head norm weights [d] (null = none)
  const float* k_gamma;
  float norm_eps;
  int norm_plus_one;
  __nv_bfloat16* k_cache;        // [B, nkv, Tmax, d]; position pos is appended
  __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [B, nh d]
  const int64_t* pos_dev;        // position of the new token, read on the device when non-null
  int64_t pos0, Tmax, B;
  int nh, nkv, d;
  int64_t window;                // 0 = none
  float softcap;                 // 0 = none
  int splits;                    // grid z = cluster size: context slices per (row, kv head)
  int push_merge;                // set by the launcher: the slices' partials are pushed to the finishing CTA
};
// Rope + cache append + attention + merge of one new token per row, in one launch.
int k_launch_attn_dec(cg_ctx* c, const AttnDecArgs& a);
int attn_dec_splits(int64_t Tmax, int64_t pairs, int d);

// tokens[b] = argmax over the vocabulary with the reference's tie rule (last index); optional
// soft-cap applied to the logits in place first.  The logits are `parts` vocabulary slices of
// Vp entries laid out [parts, B, Vp] (parts = 1: plain [B, V]).  Also appends the token to
// history[b * hist_ld + n] where n = *count_dev (a device counter) and, if advance != 0,
// increments *count_dev and *pos_dev afterwards.  `best` is B zeroed 64-bit merge slots;
// they are zero again when the call has run.
int k_launch_argmax(cg_ctx* c, float* logits, int64_t B, int64_t Vp, int parts, float softcap, uint32_t* tokens,
                    uint32_t* history, int64_t hist_ld, int64_t* count_dev, int64_t* pos_dev, int advance,
                    unsigned long long* best);

// What a kernel needs to push an addend of a small all-reduce into every rank's exchange
// area (see PeerXchg) and what the consumer needs to collect it.
struct PeerPush {
  float* data[MAX_PEERS];
  uint32_t* flags[MAX_PEERS];
  uint32_t* epoch;
  unsigned* ticket;
  int world, rank;
  int64_t max_elems;
};
inline PeerPush peer_push_of(const PeerXchg& x) {
  PeerPush p;
  for (int r = 0; r < MAX_PEERS; ++r) { p.data[r] = x.data[r]; p.flags[r] = x.flags[r]; }
  p.epoch = x.epoch; p.ticket = x.ticket; p.world = x.world; p.rank = x.rank; p.max_elems = x.max_elems;
  return p;
}

// x[m, :] += sum over ranks (in rank order) of the addends pushed for the latest reduction,
// then out = rmsnorm(x) as k_launch_rmsnorm.  Waits (bounded) for every rank's flag first.
int k_launch_rmsnorm_reduce(cg_ctx* c, const PeerPush& px, float* x, int64_t ldx, const float* gamma, float eps, int plus_one,
                            int64_t M, int64_t H, void* out, int out_bf16);
// Tensor-parallel greedy pick: every rank reduces its own vocabulary slice [B, Vp] (global
// index = rank * Vp + i) to one candidate per row, pushes the candidates to all ranks, and
// every rank takes the best (ties -> last index) and advances its counters as k_launch_argmax.
int k_launch_argmax_tp(cg_ctx* c, const PeerPush& px, float* logits, int64_t B, int64_t Vp, float softcap, uint32_t* tokens,
                       uint32_t* history, int64_t hist_ld, int64_t* count_dev, int64_t* pos_dev, int advance,
                       unsigned long long* best);

// Weight-streaming GEMM for a handful of tokens (M <= 32): y[M, N] = x[M, K] w[N, K]^T on bf16
// activations.  The gate/up pair can share a CTA with act(gate) * up as the epilogue, and
// split-K partials are reduced inside a thread-block cluster.
struct DecGemm {
  const __nv_bfloat16* x;   // [M, K] activations with row stride ldx
  int64_t ldx;
  const __nv_bfloat16* w;   // [w_rows, K] bf16, row stride ldw
  int64_t ldw, w_rows;
  void* out;                // [M, N] with row stride ldo
  int64_t ldo;
  const float* residual;
  int out_mode;             // 0: f32, 1: bf16, 2: f32 out = product + residual,
                            // 3: the product is pushed as this rank's addend of an all-reduce (out unused)
  const PeerPush* push;     // for out_mode 3
  // Norm hand-over between consecutive GEMMs (RMSNorm(x) W^T = (x g) W^T / rms(x) row by row):
  // a residual GEMM (out_mode 2) that is followed by a norm can also write xb_out = bf16(out * g)
  // (g = g_next, or 1 + g_next) and ss_out[part][32] = per-CTA sums of out^2 per token; the GEMM
  // after the norm then reads xb as its activations and multiplies row m of its accumulators by
  // 1 / sqrt(sum_parts ss_in[part][m] / K + ss_eps).  All null / zero = off.
  __nv_bfloat16* xb_out = nullptr;
  const float* g_next = nullptr;
  int g_plus_one = 0;
  float* ss_out = nullptr;
  const float* ss_in = nullptr;
  int ss_parts = 0;
  float ss_eps = 0.f;
  int dual;                 // 1: rows n and n + N of w form gate and up; out = act(gate) * up
  int act;                  // 0 silu, 1 tanh-gelu
  int64_t M, N, K;
};
int gemm_dec(cg_ctx* c, const DecGemm& g);
int gemm_dec_ss_parts(int64_t N, int64_t K);  // partials per token a hand-over producer with this shape writes
bool gemm_dec_supported(int64_t M, int64_t K);

// Mixture-of-experts feed-forward block (catgrad-llm/src/models/qwen3.rs:64-133) on M tokens:
// x += sum over the top-k experts of weight * down(act(gate(xn)) * up(xn)), xn = rmsnorm(x).
struct MoeWork {              // device scratch for up to `pairs` (token, slot) pairs
  uint32_t* ids;              // [pairs] expert of each pair, token-major
  float* wts;                 // [pairs] routing weight of each pair
  int32_t* pos;               // [pairs] row of the pair in grouped order, -1 = not on this rank
  int32_t *tile_expert, *tile_row0, *tile_rows, *n_tiles;  // GEMM tile list ([pairs] each, one count)
  __nv_bfloat16* xg;          // [pairs, H] activations in grouped order
  __nv_bfloat16* h;           // [pairs, Fe]
  float* y;                   // [pairs, H]
};
struct MoeArgs {
  const float* x;             // [M, H] input rows (the residual stream)
  float* out;                 // [M, H] result; may be x
  const float* gamma;         // norm weights [H]; null = x is used as it is
  float eps;
  int plus_one;
  const float* router;        // [E, H] f32 (used when router3 is null)
  const __nv_bfloat16* router3;  // [E, 3 H] bf16: the router matrix three times along k, or null
  __nv_bfloat16* xs3;         // [M, 3 H] scratch for router3
  float* logits;              // [M, E] scratch for router3
  const __nv_bfloat16 *w_gate, *w_up;  // [El, Fe, H] experts this rank owns
  const __nv_bfloat16* w_down;         // [El, H, Fe]
  int H, E, k, Fe, norm_topk, act;
  int e_lo, El;               // this rank owns experts [e_lo, e_lo + El)
  int add_residual;           // 1: out = x + expert sum; 0: out = this rank's expert sum only
  const PeerPush* push = nullptr;  // tensor-parallel decode: x (= out) first receives the addends pushed by the
                              // preceding row-parallel GEMM, and the expert sum is pushed as the next addend
  int64_t M;
  __nv_bfloat16* xn;          // [M, H] scratch: the normalised rows
  MoeWork w;
};
int moe_ffn(cg_ctx* c, const MoeArgs& a);
int moe_pick_tn(int64_t pairs, int experts);
int64_t moe_max_tiles(int64_t pairs, int experts_local, int tn);

// All decode steps of a call as one resident kernel (decode_resident.cu): dense pre-norm
// decoders on one GPU, at most 32 rows, head size 64 or 128.
struct ResidentLayerDesc {
  const __nv_bfloat16 *w_qkv, *w_o, *w_gu, *w_down;  // [(nh + 2 nkv) d, H], [H, nh d], [2 F, H], [H, F]
  const float *gain_in, *gain_ffn;                    // input norm, pre-FFN norm
  const float *q_gamma, *k_gamma;                     // per-head norms or null
  const float *cos_t, *sin_t;                         // rotary tables [Tmax, d / 2]
  __nv_bfloat16 *k_cache, *v_cache;                   // [B, nkv, Tmax, d]
  int64_t window;                                     // 0 = none
};
struct ResidentModel {
  std::vector<ResidentLayerDesc> layers;
  const __nv_bfloat16* head;   // [Vp, H]
  const float* gain_final;
  const void* embed;           // [vocab, H] f32 or bf16
  int embed_storage;
  int64_t H, F, Vp, vocab, Tmax;
  int nh, nkv, d, act, plus_one;
  float eps, attn_softcap, final_softcap, embed_scale;
  // workspace of the decoder (all device pointers)
  float* x;                    // [M, H] residual stream
  __nv_bfloat16* xn;           // [M, H]
  float* ss;                   // [ss_parts_cap][32] partial sums of squares (used as two halves)
  int64_t ss_parts_cap;
  float* qkv;                  // [M, (nh + 2 nkv) d]
  __nv_bfloat16* att;          // [M, nh d]
  __nv_bfloat16* hact;         // [M, F]
  float* logits;               // [M, Vp]
  uint32_t* cur;               // [M] tokens of the next step
  uint32_t* history;
  int64_t hist_ld;
  int64_t *count_dev, *pos_dev;
  unsigned long long* best;    // [M] zeroed 64-bit merge slots
};
struct ResidentPlan;
bool decode_resident_supported(const ResidentModel& m, int64_t M);
// Builds the static schedule, tensor maps and device tables for M rows.
int decode_resident_prepare(cg_ctx* c, const ResidentModel& m, int64_t M, ResidentPlan** out);
// Enqueues n_steps decode steps: reads the tokens in `cur`, leaves the last pick there, appends
// every pick to the history and advances the device counters by n_steps.
int decode_resident_run(cg_ctx* c, ResidentPlan* plan, int n_steps);
void decode_resident_free(ResidentPlan* plan);
int64_t decode_resident_bytes_per_step(const ResidentPlan* plan);  // weight bytes one step streams
int decode_resident_grid(const ResidentPlan* plan);                // resident CTAs
// Diagnostics: out == null arms the timeline of CTA `cta` for the next run (cta < 0 disarms);
// otherwise copies n globaltimer stamps (two per phase: may start, this CTA done) to the host.
int decode_resident_trace(cg_ctx* c, ResidentPlan* plan, int cta, uint64_t* out, int n);

// f32 -> bf16 rows (ld in elements for the source)
int k_launch_to_bf16(cg_ctx* c, const float* x, int64_t n, __nv_bfloat16* out);

}  // namespace cg
