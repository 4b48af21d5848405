/*
 * catgrad_cuda.h — C ABI of the B200-native tensor backend for the catgrad interpreter.
 *
 * The first half of this header is a 1:1 restatement of the catgrad interpreter's
 * `trait Backend` (catgrad/src/interpreter/backend/mod.rs:22-82) as `extern "C"` entry
 * points over opaque, reference-counted device tensors.  Each entry point cites the trait
 * method it replaces.  Conventions carried over from the trait (backend/mod.rs:16-21):
 * no implicit broadcasting, binary ops require identical shapes, reductions act on the
 * last axis and keep the rank.
 *
 * The second half ("extensions") holds what the trait cannot express because it is eager
 * and op-at-a-time: fused kernels, the bf16 tensor-core GEMM, the device KV cache and the
 * decoder runner that the benchmark drives, plus the tensor-parallel communicator.
 *
 * Ownership.  The Rust trait moves tensors into every call; in C every `cg_tensor*`
 * argument is BORROWED and every `cg_tensor**` result is a NEW reference the caller must
 * drop with cg_tensor_release.  `Clone` of the Rust wrapper = cg_tensor_retain (O(1)).
 *
 * Errors.  Every call returns a cg_status (0 = ok).  The library never aborts the
 * process; the message for the last failure on a context is cg_last_error(ctx).  The
 * reference backends panic on the same conditions (ndarray.rs:212,255,293,333;
 * candle.rs:413-415 "Shape mismatch in operation"); a Rust shim turns a non-zero status
 * into the same panic.
 *
 * Threading.  A context owns one CUDA stream; calls on one context must not overlap.
 * All work is enqueued on that stream; only cg_to_vec_*, cg_compare and cg_sync block.
 * cg_shape / cg_dtype answer from host metadata and never synchronise
 * (BackendTensorOps::shape, backend/mod.rs:84-86).
 *
 * Dtype tags.  The interpreter knows F32 and U32 only (catgrad/src/category/core.rs:21-24).
 * With precision CG_PREC_BF16 the backend may STORE an F32-tagged tensor as bf16 (weights
 * uploaded through cg_ndarray_from_vec_f32 with rank >= 2); cg_to_vec_f32 always returns f32.
 */
#ifndef CATGRAD_CUDA_H
#define CATGRAD_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CG_MAX_RANK 8

typedef struct cg_ctx cg_ctx;
typedef struct cg_tensor cg_tensor;
typedef struct cg_decoder cg_decoder;

typedef enum cg_status {
  CG_OK = 0,
  CG_ERR_SHAPE = 1,       /* BackendError::ShapeError / "Shape mismatch in operation" */
  CG_ERR_DTYPE = 2,       /* e.g. sin on U32 ("Invalid input types for sin") */
  CG_ERR_INVALID = 3,     /* null pointer, bad dim, bad k ... */
  CG_ERR_CUDA = 4,        /* a CUDA runtime call failed; message has the CUDA error string */
  CG_ERR_OOM = 5,
  CG_ERR_INDEX = 6,       /* an index tensor held a value >= the indexed dimension */
  CG_ERR_TIMEOUT = 7,     /* a bounded device-side wait expired */
  CG_ERR_UNSUPPORTED = 8,
  CG_ERR_COMM = 9
} cg_status;

typedef enum cg_dtype { CG_F32 = 0, CG_U32 = 1 } cg_dtype;           /* core.rs:21-24 */
typedef enum cg_precision { CG_PREC_F32 = 0, CG_PREC_BF16 = 1 } cg_precision;

/* ------------------------------------------------------------------ context ---------- */

/* Create a backend on CUDA device `device`.  `stream` is a cudaStream_t to enqueue on, or
 * NULL to let the context create its own.  Stands where `NdArrayBackend` /
 * `CandleBackend::new()` are constructed (backend/candle.rs:36-60). */
int32_t cg_ctx_create(int32_t device, int32_t precision, void* stream, cg_ctx** out);
int32_t cg_ctx_destroy(cg_ctx* ctx);
const char* cg_last_error(cg_ctx* ctx);
/* Block until everything enqueued so far has run; also surfaces device-side error flags
 * (CG_ERR_INDEX, CG_ERR_TIMEOUT) raised by earlier kernels. */
int32_t cg_sync(cg_ctx* ctx);
/* The cudaStream_t the context enqueues on (for event timing by the caller). */
void* cg_ctx_stream(cg_ctx* ctx);
/* Number of kernels this library has launched on the context since creation. */
int64_t cg_launch_count(cg_ctx* ctx);
/* Bytes currently held from the device by the context's caching allocator. */
int64_t cg_bytes_reserved(cg_ctx* ctx);

/* ------------------------------------------------------------------ handles ---------- */

int32_t cg_tensor_retain(cg_tensor* t);     /* Clone of BackendTensor */
int32_t cg_tensor_release(cg_tensor* t);    /* Drop of BackendTensor */
/* BackendTensorOps::shape (backend/mod.rs:84-86).  Writes rank and dims[0..rank). */
int32_t cg_shape(const cg_tensor* t, int32_t* rank, int64_t dims[CG_MAX_RANK]);
/* TaggedTensorTuple::dtype (interpreter/types.rs:15-98): the tag, CG_F32 or CG_U32. */
int32_t cg_dtype_of(const cg_tensor* t, int32_t* dtype);

/* ------------------------------------------------------ trait Backend, method by method */

/* Backend::zeros (mod.rs:26; ndarray.rs:53-65) */
int32_t cg_zeros(cg_ctx*, const int64_t* dims, int32_t rank, int32_t dtype, cg_tensor** out);
/* Backend::ndarray_from_vec_f32 (mod.rs:28-32; ndarray.rs:67-77).  `n` must equal the
 * product of dims, else CG_ERR_SHAPE (BackendError::ShapeError). */
int32_t cg_ndarray_from_vec_f32(cg_ctx*, const float* data, int64_t n, const int64_t* dims,
                                int32_t rank, cg_tensor** out);
/* Backend::ndarray_from_vec_u32 (mod.rs:34-38; ndarray.rs:79-89) */
int32_t cg_ndarray_from_vec_u32(cg_ctx*, const uint32_t* data, int64_t n, const int64_t* dims,
                                int32_t rank, cg_tensor** out);
/* Backend::cast (mod.rs:40; ndarray.rs:97-114): f32->u32 saturates, NaN->0; u32->f32 rounds */
int32_t cg_cast(cg_ctx*, const cg_tensor* x, int32_t dtype, cg_tensor** out);
/* Backend::matmul (mod.rs:41; ndarray.rs:116-122, 531-615): rank>=2, batch dims equal */
int32_t cg_matmul(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
/* Backend::add/sub/mul/div (mod.rs:42-45; ndarray.rs:124-154, 401-431).  u32 wraps;
 * u32 division by zero yields 0xFFFFFFFF (the reference panics). */
int32_t cg_add(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
int32_t cg_sub(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
int32_t cg_mul(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
int32_t cg_div(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
/* Backend::pow (mod.rs:46; ndarray.rs:156-162, 443-453): f32 powf, u32 wrapping pow */
int32_t cg_pow(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
/* Backend::lt / eq (mod.rs:47-48; ndarray.rs:164-198): result is 1/0 in the INPUT dtype */
int32_t cg_lt(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
int32_t cg_eq(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
/* Backend::sin / cos (mod.rs:49-50; ndarray.rs:208-222): F32 only, else CG_ERR_DTYPE */
int32_t cg_sin(cg_ctx*, const cg_tensor* x, cg_tensor** out);
int32_t cg_cos(cg_ctx*, const cg_tensor* x, cg_tensor** out);
/* Backend::neg (mod.rs:51; ndarray.rs:200-206, 433-441): u32 = wrapping negation */
int32_t cg_neg(cg_ctx*, const cg_tensor* x, cg_tensor** out);
/* Backend::broadcast (mod.rs:52; ndarray.rs:259-265, 355-361): `dims` is the full target
 * shape, right-aligned numpy rule.  Returns a stride-0 view (no kernel). */
int32_t cg_broadcast(cg_ctx*, const cg_tensor* x, const int64_t* dims, int32_t rank, cg_tensor** out);
/* Backend::reshape (mod.rs:53; ndarray.rs:311-317, 347-353): logical row-major order */
int32_t cg_reshape(cg_ctx*, const cg_tensor* x, const int64_t* dims, int32_t rank, cg_tensor** out);
/* Backend::transpose (mod.rs:54; ndarray.rs:267-273, 363-371): swap two axes (view) */
int32_t cg_transpose(cg_ctx*, const cg_tensor* x, int32_t dim0, int32_t dim1, cg_tensor** out);
/* Backend::max (mod.rs:55; ndarray.rs:224-230, 455-467): fold from f32::MIN with a
 * NaN-ignoring max (so an all -inf row gives f32::MIN); u32 from 0 */
int32_t cg_max(cg_ctx*, const cg_tensor* x, cg_tensor** out);
/* Backend::sum (mod.rs:56; ndarray.rs:232-238, 522-529) */
int32_t cg_sum(cg_ctx*, const cg_tensor* x, cg_tensor** out);
/* Backend::argmax (mod.rs:57; ndarray.rs:240-246, 469-493): u32 index, IEEE total order,
 * ties -> LAST index */
int32_t cg_argmax(cg_ctx*, const cg_tensor* x, cg_tensor** out);
/* Backend::topk (mod.rs:58; ndarray.rs:248-257, 495-520): stable descending sort by total
 * order, ties -> LOWER index first.  F32 only. */
int32_t cg_topk(cg_ctx*, const cg_tensor* x, int64_t k, cg_tensor** values, cg_tensor** indices);
/* Backend::compare (mod.rs:59; ndarray.rs:337-343): same shape and all elements == */
int32_t cg_compare(cg_ctx*, const cg_tensor* a, const cg_tensor* b, int32_t* equal);
/* Backend::concat (mod.rs:60-65; ndarray.rs:319-335, 393-399) */
int32_t cg_concat(cg_ctx*, const cg_tensor* a, const cg_tensor* b, int32_t dim, cg_tensor** out);
/* Backend::index (mod.rs:66-71; ndarray.rs:275-295, 373-381): select along `dim`;
 * indices (U32, any rank) are flattened */
int32_t cg_index(cg_ctx*, const cg_tensor* x, int32_t dim, const cg_tensor* indices, cg_tensor** out);
/* Backend::slice (mod.rs:72-78; ndarray.rs:297-309, 383-391): offset view */
int32_t cg_slice(cg_ctx*, const cg_tensor* x, int32_t dim, int64_t start, int64_t len, cg_tensor** out);
/* Backend::arange (mod.rs:79; ndarray.rs:91-95): U32 [0, end) built through f32 */
int32_t cg_arange(cg_ctx*, int64_t end, cg_tensor** out);
/* Backend::to_vec (mod.rs:81; ndarray.rs:46-51).  `n` = capacity in elements; must be the
 * tensor's element count.  Blocks.  A strided view is gathered first (the reference
 * panics on non-standard layout). */
int32_t cg_to_vec_f32(cg_ctx*, const cg_tensor* x, float* dst, int64_t n);
int32_t cg_to_vec_u32(cg_ctx*, const cg_tensor* x, uint32_t* dst, int64_t n);

/* ------------------------------------------------------------------ extensions ------- */

/* Runtime switches (name, value):
 *   "gemm"  : 0 = auto (tcgen05 bf16 when an operand is stored bf16, else f32 SIMT),
 *             1 = force the f32 SIMT kernel (cross-check path for tests)
 *   "pdl"   : 1 (default) = fused kernels are launched with programmatic stream serialization
 *   "persistent" : 1 (default) = GEMMs with several output tiles per SM run as one resident
 *             CTA per SM with double-buffered accumulators; 0 = one CTA per tile
 *   "pair_cta" : 1 (default) = among those, GEMMs with several 256 x 256 tiles per SM pair run on
 *             thread-block clusters of two CTAs (tcgen05 cta_group::2: one 256 x 256 tile per pair,
 *             each CTA loading its own weight rows and half of the activation tile); 2 = every
 *             tensor-core GEMM without a k split does (tests); 0 = never
 *   "handover" : 1 (default) = in decode steps of pre-norm models the residual GEMMs also leave
 *             the gain-scaled bf16 activations and per-row sums of squares, and the next GEMM
 *             applies 1 / rms in its epilogue (no separate norm kernel); 0 = norm kernels
 *   "fa"    : 1 (default) = prefill attention on tcgen05 / TMEM for head sizes 64 and 128 without
 *             soft-cap or window (2 = its 64-key-tile variant); 0 = the mma.sync kernel everywhere
 *   "prefill_chunk" : tokens per prefill chunk (default 8192; bounds the decoder's workspace)
 *   "peer"  : 1 (default) = decode steps under tensor parallelism reduce over mapped peer
 *             memory (see cg_comm_peer_exchange); 0 = NCCL collectives.  Set before the first
 *             decode step, and identically on every rank.
 *   "resident" : 1 = decode steps of dense pre-norm models on one GPU run as ONE resident kernel
 *             for all requested steps (one CTA per SM, phases separated by bounded grid barriers,
 *             weights streamed through a shared-memory ring that keeps filling across phase
 *             boundaries); 0 (default) = one kernel per operation, captured into a CUDA graph.
 *             Both give the same logits within bf16 rounding; the per-operation path is the
 *             faster one at the measured shapes, so it stays the default.
 *   "lazy"  : 1 = the trait methods are RECORDED instead of run (binary ops, neg, cast, max, sum,
 *             matmul, concat, arange and the views): each returns a handle with shape and dtype
 *             whose contents do not exist yet.  When contents are needed -- cg_to_vec_*,
 *             cg_compare, a method that is not recorded (sin, cos, eq, argmax, topk, index),
 *             cg_sync, or any entry point outside the trait -- the recorded calls run in order,
 *             with the chains catgrad's stdlib and model graphs lower to replaced by one fused
 *             kernel each: rmsnorm (helpers.rs:120-145), softmax (nn/mod.rs:162-171),
 *             silu(g) * u (nn/mod.rs:146-148), rope (helpers.rs:202-221) and the attention core
 *             (models/llama.rs:97-108) seen through repeat_kv and the causal mask, so that the
 *             S x S scores never exist.  A value inside a chain is skipped only when nothing else
 *             reads it and the caller holds no handle to it.  Results equal eager mode's within
 *             f32 rounding (integer and index results exactly); errors a recorded call would
 *             raise for its shapes or dtypes are raised when it is recorded.  0 (default) = eager.
 *             Setting it to 0 first runs what is pending.
 *   "resident_attn_group" : CTAs that share one (row, kv head) in the resident kernel's attention
 *             phase: 1, 2 or 4; 0 (default) = chosen from the batch and the cache length
 *   "wait_limit_us" : limit of every bounded device-side wait (default 1 000 000).  When a wait
 *             runs out the kernel gives up, later waits of the context give up at once, and the
 *             next cg_sync returns CG_ERR_TIMEOUT and clears the condition.
 * A decoder re-captures its decode-step graph after any option change.
 */
int32_t cg_set_option(cg_ctx*, const char* name, int64_t value);

/* Counters of the deferred-evaluation mode: trait calls recorded so far, chains replaced by a
 * fused kernel so far, calls currently pending.  No counterpart in the reference. */
int32_t cg_lazy_stats(cg_ctx*, int64_t* recorded, int64_t* fused, int64_t* pending);

/* Failure-path probe: enqueues one small kernel that waits (bounded by "wait_limit_us") on a
 * flag of the context that nothing ever raises.  The wait runs out, the kernel returns, and the
 * next cg_sync reports CG_ERR_TIMEOUT; the context stays usable.  Nothing faults or traps.
 * No counterpart in the reference (its backends have no device-side waits). */
int32_t cg_probe_wait_timeout(cg_ctx*);

/* Storage precision of a tensor: 0 = f32, 1 = u32, 2 = bf16 (F32 tag stored as bf16). */
int32_t cg_storage_of(const cg_tensor* t, int32_t* storage);
/* Round an F32-tagged tensor to bf16 storage / widen it back (new tensor). */
int32_t cg_to_bf16(cg_ctx*, const cg_tensor* x, cg_tensor** out);
int32_t cg_to_f32(cg_ctx*, const cg_tensor* x, cg_tensor** out);

/* Fused kernels.  Each computes what the cited op chain of the reference computes, in one
 * launch, on contiguous row-major inputs. */

/* rmsnorm(x) = x / pow(sum(x*x)/n + eps, 0.5) * gamma   (catgrad-llm/src/helpers.rs:120-145);
 * plus_one != 0 multiplies by (1 + gamma) instead (catgrad-llm/src/models/gemma3.rs:60-68).
 * x: [..., n] F32, gamma: [n]. */
int32_t cg_fused_rmsnorm(cg_ctx*, const cg_tensor* x, const cg_tensor* gamma, float eps,
                         int32_t plus_one, cg_tensor** out);
/* softmax over the last axis (catgrad/src/stdlib/nn/mod.rs:162-171); softcap > 0 first
 * maps x -> softcap * tanh(x / softcap) (tanh as in nn/mod.rs:138-144). */
int32_t cg_fused_softmax(cg_ctx*, const cg_tensor* x, float softcap, cg_tensor** out);
/* act(gate) * up with act = silu (0) or tanh-approx gelu (1)
 * (nn/mod.rs:146-160; models/llama.rs:27; models/gemma3.rs:28). */
int32_t cg_fused_act_mul(cg_ctx*, const cg_tensor* gate, const cg_tensor* up, int32_t act,
                         cg_tensor** out);
/* cos*x + sin*rotate_half(x) for x [b, heads, s, d] at positions pos0..pos0+s
 * (catgrad-llm/src/helpers.rs:164-221); tables are computed from theta as rope_tables does. */
int32_t cg_fused_rope(cg_ctx*, const cg_tensor* x, float theta, int64_t pos0, cg_tensor** out);
/* softmax(q k^T / sqrt(d) + causal mask) v for q [b, nh, s, d], k,v [b, nkv, s, d] with
 * grouped heads as repeat_kv orders them (helpers.rs:147-161; models/llama.rs:97-108).
 * window > 0 additionally masks keys more than window-1 positions behind the query;
 * softcap > 0 soft-caps the scaled scores. */
int32_t cg_fused_attention(cg_ctx*, const cg_tensor* q, const cg_tensor* k, const cg_tensor* v,
                           int64_t window, float softcap, cg_tensor** out);
/* y = x W^T for x [..., in] and a weight W [out, in] as stored by the checkpoints
 * (linear_no_bias, nn/mod.rs:174-199), without materialising the transpose.  Uses the
 * tcgen05 kernel when W is stored bf16. */
int32_t cg_linear(cg_ctx*, const cg_tensor* x, const cg_tensor* w, cg_tensor** out);
/* The gated half of an FFN in one kernel (catgrad-llm/src/models/llama.rs:24-28): for a
 * bf16-stored weight [2F, in] whose first F rows are the gate projection and whose last F rows
 * are the up projection, y = act(x Wg^T) * (x Wu^T), rounded once to bf16 storage.  act: 0 silu,
 * 1 tanh gelu.  The [.., 2F] intermediate is never written. */
int32_t cg_linear_glu(cg_ctx*, const cg_tensor* x, const cg_tensor* w, int32_t act, cg_tensor** out);
/* A tensor of independent N(mean, std) samples generated on the device (counter-based, a
 * function of seed and element index only).  Stored like an upload of the same shape (bf16
 * for rank >= 2 under CG_PREC_BF16).  No counterpart in the reference, whose weights always
 * come from a checkpoint; this exists so that multi-gigabyte synthetic checkpoints need not
 * cross the host link. */
int32_t cg_randn(cg_ctx*, const int64_t* dims, int32_t rank, uint64_t seed, float mean, float std,
                 cg_tensor** out);
/* The mixture-of-experts block of catgrad-llm/src/models/qwen3.rs:64-133 on rows x [.., H]
 * (already normalised): softmax(x router^T) -> top_k experts per row (ties -> lower id, as
 * Backend::topk) -> weights renormalised to sum 1 when norm_topk != 0 -> out = sum over the
 * chosen experts (in slot order) of weight * down_e(act(gate_e x) * up_e x).  router [E, H],
 * gate/up [E, F, H], down [E, H, F] as the checkpoints stack them.  The expert matmuls run on
 * the tensor cores with bf16 operands; routing is f32.  ids_out (optional) receives the chosen
 * expert ids [rows, top_k] U32. */
int32_t cg_fused_moe(cg_ctx*, const cg_tensor* x, const cg_tensor* router, const cg_tensor* gate,
                     const cg_tensor* up, const cg_tensor* down, int32_t top_k, int32_t norm_topk,
                     int32_t act, cg_tensor** out, cg_tensor** ids_out);

/* --- decoder runner: the greedy loop of catgrad-llm/examples/llama/main.rs:118-169 with a
 * device KV cache (cache semantics of catgrad-llm/src/legacy/models/utils.rs:210-228). --- */

typedef struct cg_decoder_config {
  int32_t arch;             /* 0 = llama (models/llama.rs), 1 = qwen3 (models/qwen3.rs),
                               2 = gemma-2-shaped (models/gemma3.rs graph + soft-caps + window) */
  int32_t num_layers;
  int32_t hidden;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t ffn;
  int32_t vocab;
  float rms_eps;
  float rope_theta;
  int32_t tie_embeddings;
  int32_t max_seq;          /* capacity of the KV cache in positions */
  int32_t max_batch;
  /* architecture switches (0 / 0.0 = off) */
  int32_t qk_norm;          /* per-head RMSNorm on q and k (qwen3.rs:187-217) */
  int32_t act;              /* 0 silu, 1 tanh-gelu */
  int32_t norm_plus_one;    /* (1 + gamma) norms (gemma3.rs:60-68) */
  int32_t post_norms;       /* post-attention and post-ffn norms (gemma3.rs:192-238) */
  float embed_scale;        /* 0 = none, else multiply embeddings (gemma3.rs:257-260) */
  float attn_softcap;
  float final_softcap;
  int32_t sliding_window;   /* 0 = none */
  int32_t window_every;     /* layers with (i % window_every) != window_every-1 use the window */
  /* frequency rescaling of long-context checkpoints (legacy/nn/rope.rs:32-201; legacy/models/utils.rs:19-48) */
  int32_t rope_scaling;     /* 0 = none, 1 = "llama3", 2 = "yarn" */
  float rope_factor;
  float rope_low_freq_factor;   /* llama3 */
  float rope_high_freq_factor;  /* llama3 */
  float rope_beta_fast;         /* yarn */
  float rope_beta_slow;         /* yarn */
  int32_t rope_original_max_pos;
  float rope_local_theta;   /* 0 = one rope base; else the base of "local" layers (gemma3.rs:154-159) */
  int32_t rope_local_every; /* layers with (i + 1) % rope_local_every != 0 rotate with rope_local_theta,
                               the others with rope_theta (the reference's sliding_window_pattern) */
  /* mixture of experts (qwen3.rs:64-133): a layer whose checkpoint carries a router
   * ("...mlp.gate.weight" [n_experts, hidden]) and stacked experts
   * ("...mlp.experts.{gate,up,down}_proj.weight") runs the expert block instead of the dense FFN */
  int32_t n_experts;        /* 0 = dense FFN everywhere; at most 1024 */
  int32_t top_k;            /* experts per token, 1..32 */
  int32_t moe_ffn;          /* width of one expert */
  int32_t norm_topk;        /* renormalise the top-k probabilities to sum 1 */
  /* tensor parallelism: this rank's place; 1 rank = no communication.  Heads, dense FFN columns
   * and the vocabulary are split over the ranks (fewer kv heads than ranks: kv heads are
   * replicated), whole experts are owned by ranks. */
  int32_t tp_rank;
  int32_t tp_world;
  /* expert parallelism with data-parallel attention (qwen3.rs:64-133 sharded over ranks; needs
   * tp_world = 1 and cg_comm_init): every rank holds the dense weights whole and n_experts /
   * ep_world experts, runs ITS OWN batch rows (the caller hands each rank its rows), and on every
   * expert layer the rows of all ranks are all-gathered, routed identically everywhere (f32),
   * run through the experts this rank owns, and the expert sums reduce-scattered back to the
   * rows' owners.  With top-8 of 128 experts on 8 ranks a token visits nearly every rank, so
   * this moves the bytes an all-to-all dispatch / combine would.  0 or 1 = off. */
  int32_t ep_rank;
  int32_t ep_world;
} cg_decoder_config;

int32_t cg_decoder_create(cg_ctx*, const cg_decoder_config* cfg, cg_decoder** out);
int32_t cg_decoder_destroy(cg_decoder*);
/* Hand over one checkpoint tensor by its Hugging Face name (the names the reference
 * splits on '.', examples/llama/main.rs:325), e.g. "model.layers.0.self_attn.q_proj.weight".
 * Full (unsharded) tensors are passed on every rank; the decoder keeps its shard. */
int32_t cg_decoder_set_param(cg_decoder*, const char* name, const cg_tensor* t);
/* Hand over every tensor of a .safetensors checkpoint file (replaces the host-side load of
 * examples/llama/main.rs:279-354: there every tensor is widened to a host Vec<f32> first; here the
 * file is memory-mapped and each tensor crosses the host link once in its stored element type,
 * F32 or BF16, anything else is refused like the reference's loader does).  Per-expert matrices
 * "model.layers.L.mlp.experts.E.{gate,up,down}_proj.weight" are placed directly into the stacked
 * [n_experts, rows, cols] tensors the expert block reads (examples/llama/main.rs:173-264 builds
 * those by repeated concatenation).  May be called once per shard file, before finalize. */
int32_t cg_decoder_load_safetensors(cg_decoder*, const char* path);
/* Build fused weights, rope tables, workspace and TMA descriptors.  Call once after all
 * parameters are set. */
int32_t cg_decoder_finalize(cg_decoder*);
/* Forget all cached positions. */
int32_t cg_decoder_reset(cg_decoder*);
/* Run the prompt: tokens is a DEVICE U32 tensor [B, S].  Fills the KV cache for positions
 * [0, S) and leaves the greedy next token of every row in the decoder's token buffer.
 * If logits_out != NULL it receives an F32 tensor [B, V] with the last position's logits. */
int32_t cg_decoder_prefill(cg_decoder*, const cg_tensor* tokens, cg_tensor** logits_out);
/* Continue a cached sequence: tokens is a DEVICE U32 tensor [B, S] (B as cached) that is run at
 * cache positions [cached, cached + S) on top of what prefill / decode / earlier appends left,
 * and the greedy next token of every row is left in the token buffer (as after prefill).  With
 * cg_decoder_truncate this is the prefix reuse of the reference's serving runner
 * (catgrad-llm/src/run.rs:282-305 keeps its KV cache when the new context extends the old one;
 * here any common prefix is kept).  cg_decoder_truncate forgets the cached positions from
 * `positions` on and clears the record of generated tokens; cg_decoder_position reports how many
 * positions are cached and how many tokens have been generated since the last prefill/truncate. */
int32_t cg_decoder_append(cg_decoder*, const cg_tensor* tokens, cg_tensor** logits_out);
int32_t cg_decoder_truncate(cg_decoder*, int64_t positions);
int32_t cg_decoder_position(cg_decoder*, int64_t* cached, int64_t* generated);
/* Advance every row by `steps` greedy tokens, feeding each step's argmax to the next with
 * no host round trip.  If logits_out != NULL, receives the last step's logits [B, V]. */
int32_t cg_decoder_decode(cg_decoder*, int32_t steps, cg_tensor** logits_out);
/* Advance by exactly one step with the given DEVICE U32 tokens [B] instead of the
 * decoder's own argmax (teacher forcing, for parity checks). */
int32_t cg_decoder_step_with(cg_decoder*, const cg_tensor* tokens, cg_tensor** logits_out);
/* Tokens generated so far as a device U32 tensor [B, n_generated] (prefill's token first). */
int32_t cg_decoder_tokens(cg_decoder*, cg_tensor** out);
/* The call the reference's example driver makes, end to end, with HOST buffers: copies
 * `prompt` [B*S] to the device, prefills, then enqueues n_decode steps back to back (the device
 * feeds each step's arg-max to the next, where the reference's host loop reads every token back
 * with to_vec, examples/llama/main.rs:160) and reads the token history back in one strided
 * device-to-host copy at the end.  `out` receives [B, 1 + n_decode] tokens. */
int32_t cg_decoder_generate(cg_decoder*, const uint32_t* prompt, int32_t batch, int32_t seq,
                            int32_t n_decode, uint32_t* out);

/* Measurement hook: enqueue only the weight-streaming GEMMs of one decode step for `batch`
 * rows (every layer's qkv, o, gate/up, down projections and the LM head, on the decoder's
 * own weights) `iters` times, timed with CUDA events on the context's stream. */
int32_t cg_decoder_time_gemms(cg_decoder*, int32_t batch, int32_t iters, float* ms_per_sweep,
                              int32_t* launches_per_sweep);

/* Diagnostics: a device-side timeline of the decode GEMM launches.  After cg_trace_enable(ctx, 1)
 * every launch records, in launch order (slot = launch number mod 2048), four globaltimer
 * stamps in nanoseconds: first CTA started, preceding kernel complete, last accumulator
 * ready, last CTA finished.  cg_trace_read copies `slots` x 4 values. */
int32_t cg_trace_enable(cg_ctx*, int32_t on);
int32_t cg_trace_read(cg_ctx*, uint64_t* out, int32_t slots);

/* Rotary tables cos, sin [T, d/2] as the runner builds them: the plain formula of
 * catgrad-llm/src/helpers.rs:164-193 (kind 0) or with the "llama3" (kind 1) / "yarn" (kind 2)
 * frequency rescaling of catgrad-llm/src/legacy/nn/rope.rs:32-201.  Unused factors are ignored. */
int32_t cg_rope_tables(cg_ctx*, float theta, int32_t kind, float factor, float low_freq_factor, float high_freq_factor,
                       float beta_fast, float beta_slow, int32_t original_max_pos, int64_t T, int64_t d,
                       cg_tensor** cos_out, cg_tensor** sin_out);

/* Diagnostics of the resident decode kernel ("resident" option): out == NULL arms a timeline of
 * resident CTA `cta` for the next decode call (cta < 0 disarms); otherwise copies n globaltimer
 * stamps in nanoseconds, two per phase of the schedule (embed, then per layer qkv GEMM,
 * attention, o GEMM, gate/up GEMM, down GEMM, then the LM head; next step likewise): when the
 * phase's grid barrier let the CTA through, and when the CTA finished its part of the phase. */
int32_t cg_decoder_resident_trace(cg_decoder*, int32_t cta, uint64_t* out, int32_t n);

/* --- .safetensors checkpoint files (examples/llama/main.rs:296-330 reads them through the
 * safetensors and memmap2 crates).  cg_safetensors_open memory-maps the file and parses its
 * header on the host (no device needed); cg_safetensors_tensor uploads tensor i as a tensor of the
 * context: F32 data as cg_ndarray_from_vec_f32 would, BF16 data without widening on the host
 * (kept as bf16 storage for rank >= 2 in a bf16-precision context, widened on the device
 * otherwise).  `storage` in cg_safetensors_info: 0 = F32, 2 = BF16.  On failure
 * cg_safetensors_open writes the reason to `err` (optional). --- */
typedef struct cg_safetensors cg_safetensors;
int32_t cg_safetensors_open(const char* path, cg_safetensors** out, char* err, int64_t err_cap);
int32_t cg_safetensors_close(cg_safetensors*);
int64_t cg_safetensors_count(const cg_safetensors*);
int32_t cg_safetensors_info(const cg_safetensors*, int64_t i, const char** name, int32_t* storage, int32_t* rank,
                            int64_t dims[CG_MAX_RANK]);
int32_t cg_safetensors_tensor(cg_ctx*, const cg_safetensors*, int64_t i, cg_tensor** out);

/* Row-wise arg-max for callers that cannot allocate device memory (code that runs while
 * another stream of the process is being captured into a CUDA graph, plugins with a fixed memory
 * budget, latency-critical loops).  It has no counterpart in the reference: it is the arg-max of
 * cg_argmax (ties -> last index, IEEE total order) on raw device pointers, with its per-row
 * merge slots in a fixed array inside the library instead of memory from an allocator.
 *   logits : device, f32 [rows, n] contiguous      out : device, u32 [rows]
 *   rows <= CG_NOALLOC_MAX_ROWS, else CG_ERR_INVALID with a message in `err` (optional buffer).
 * The call enqueues on `stream` (a cudaStream_t, NULL = default stream) of the CURRENT device and
 * calls no cudaMalloc / cudaFree.  The first call on a device resolves the array's device
 * address; make it before any stream capture.  All calls share the array: calls that overlap
 * on the GPU race; calls on one stream are safe. */
#define CG_NOALLOC_MAX_ROWS 4096
int32_t cg_argmax_rows_noalloc(void* stream, const float* logits, int64_t rows, int64_t n, uint32_t* out,
                               char* err, int64_t err_cap);

/* --- tensor-parallel communicator (NCCL over NVLink; one process per GPU) --- */

/* Size in bytes of the opaque id rank 0 creates and every rank must receive. */
int32_t cg_comm_id_size(void);
int32_t cg_comm_make_id(void* id_bytes);
/* Collective: every rank calls with the same id.  Besides the NCCL communicator this maps a
 * small exchange area of every rank into every other rank (CUDA inter-process handles,
 * carried by the new communicator), used by the decoder for reductions of a few tokens:
 * the row-parallel GEMM writes its partial product straight into all ranks' areas and the
 * norm kernel that follows sums them, so a decode step makes no collective call. */
int32_t cg_comm_init(cg_ctx*, const void* id_bytes, int32_t rank, int32_t world);
/* 1 when the peer exchange area is mapped on this rank (and therefore on all), else 0 with
 * the reason in `why` (the decoder then keeps to NCCL collectives). */
int32_t cg_comm_peer_exchange(cg_ctx*, char* why, int64_t why_cap);
int32_t cg_comm_destroy(cg_ctx*);
/* In-place sum all-reduce of an F32-tagged contiguous tensor (f32 or bf16 storage). */
int32_t cg_comm_all_reduce(cg_ctx*, cg_tensor* t);

#ifdef __cplusplus
}
#endif
#endif /* CATGRAD_CUDA_H */
