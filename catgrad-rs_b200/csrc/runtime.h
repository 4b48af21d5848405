// runtime.h — internal definitions shared by the translation units of libcatgrad_cuda.so:
// context (stream, caching allocator, device error word), reference-counted tensor handles
// with shape/stride views, and the helpers every entry point uses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/catgrad_cuda.h"

namespace cg {

enum Storage : int32_t { ST_F32 = 0, ST_U32 = 1, ST_BF16 = 2 };

inline size_t storage_bytes(int st) { return st == ST_BF16 ? 2 : 4; }

// Codes a kernel may leave in the context's device error word.
enum DevErr : int32_t { DEV_OK = 0, DEV_INDEX = 1, DEV_TIMEOUT = 2 };

struct Core;

// One device allocation handed out by the caching allocator.
struct Buffer {
  std::shared_ptr<Core> core;
  void* ptr = nullptr;
  size_t bytes = 0;   // size of the underlying block
  bool owned = true;  // false: memory belongs to someone else (never freed here)
  // The last bf16-rounded copy made of (a view of) this buffer as a GEMM operand, with the view
  // it was made for: q, k and v (or gate and up) read the same activations, and trait tensors
  // are never written after they are made, so the copy serves every one of them.  Whoever does
  // write a tensor in place (cg_comm_all_reduce) drops it.
  std::shared_ptr<Buffer> bf16_copy;
  int64_t bf16_key[5] = {0, 0, 0, 0, 0};  // offset, rows, cols, row stride, col stride
  ~Buffer();
};

// The part of a context that tensors keep alive: device, stream, allocator.
struct Core {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  std::mutex mu;
  std::multimap<size_t, void*> free_blocks;  // size -> ptr, reusable at once: one stream
  int64_t reserved = 0;                      // bytes obtained from cudaMalloc and not returned
  int32_t* dev_err = nullptr;                // device error word (DevErr)
  ~Core();
  void* alloc(size_t bytes, size_t* got);
  void recycle(void* p, size_t bytes);
  void trim();
};

// Peer exchange area for small all-reduces without a library call: every rank owns
// data[2][world][max_elems] f32 and flags[2][world] u32 in its own memory and maps the areas
// of all ranks.  A rank pushes its addend into slot [parity][its rank] of EVERY rank's area,
// then raises that slot's flag to the reduction's sequence number; a consumer waits for the
// `world` flags of its own area and sums the slots in rank order.  Two parities alternate so
// a fast rank's next push cannot overwrite what a slow rank still reads.
constexpr int MAX_PEERS = 8;
struct PeerXchg {
  bool ok = false;
  int world = 1, rank = 0;
  int64_t max_elems = 0;               // floats per slot
  float* data[MAX_PEERS] = {nullptr};  // base of every rank's data area (index = rank; own = local)
  uint32_t* flags[MAX_PEERS] = {nullptr};
  uint32_t* epoch = nullptr;           // local: sequence number of the last reduction this rank pushed
  unsigned* ticket = nullptr;          // local: CTAs of the pushing kernel that are done
  void* local_base = nullptr;
  void* opened[MAX_PEERS] = {nullptr};
  std::string why;                     // when !ok: what failed during set-up
};

}  // namespace cg

namespace cg { struct LazyNode; }

struct cg_ctx {
  std::shared_ptr<cg::Core> core;
  // deferred evaluation of the trait methods ("lazy" option; lazy.cu): calls are recorded as nodes
  // and run, with recognised chains replaced by fused kernels, when a result is needed
  bool lazy = false;
  bool lazy_busy = false;                 // the recorded nodes are being executed: entry points run eagerly
  std::vector<cg::LazyNode*> lazy_nodes;
  int64_t lazy_fused = 0;                 // chains replaced by a fused kernel so far
  int64_t lazy_recorded = 0;              // trait calls recorded so far
  int precision = CG_PREC_F32;
  std::string err;
  int64_t launches = 0;
  int opt_gemm = 0;       // 0 auto, 1 force f32 SIMT
  int opt_pdl = 1;        // programmatic dependent launch for the fused kernels
  int opt_persistent = 1; // large GEMMs take the persistent double-buffered kernel
  int opt_pair_cta = 1;   // 1: the largest of those take the CTA-pair (cta_group::2) kernel; 2: every GEMM that reaches gemm_tc does
  int opt_handover = 1;   // decode steps: residual GEMMs prepare the next norm, the next GEMM applies 1 / rms
  int opt_fa = 1;         // prefill attention on tcgen05 (attention_fa.cu) where it applies
  int opt_prefill_chunk = 8192;  // tokens per prefill chunk (bounds the decoder's workspace)
  int opt_peer = 1;       // small all-reduces over mapped peer memory instead of NCCL (when available)
  int opt_resident = 0;   // 1: decode steps of dense pre-norm models run as one resident kernel (decode_resident.cu)
  int opt_res_group = 0;  // resident decode: CTAs per (row, kv head) in the attention phase (0 = chosen by the library)
  int opt_res_stages = 0;  // resident decode: cap on the ring depth (0 = as deep as shared memory allows)
  int64_t opt_generation = 0;  // bumped by every cg_set_option
  bool trace_on = false;  // record a device timeline of the decode GEMM launches
  int64_t trace_next = 0;
  void* comm = nullptr;   // ncclComm_t
  int comm_rank = 0, comm_world = 1;
  cg::PeerXchg xchg;
  // host function pointer of cuTensorMapEncodeTiled, resolved on first use
  void* encode_tiled = nullptr;
};

struct cg_tensor {
  std::atomic<int> rc{1};
  cg_ctx* ctx = nullptr;
  int tag = CG_F32;            // the interpreter's dtype tag
  int storage = cg::ST_F32;    // how elements are stored
  int rank = 0;
  int64_t dims[CG_MAX_RANK] = {0};
  int64_t strides[CG_MAX_RANK] = {0};  // in elements
  int64_t offset = 0;                  // in elements
  std::shared_ptr<cg::Buffer> buf;
  // deferred evaluation: a tensor whose contents do not exist yet points at the node that will
  // produce them (buf is null until then); lazy_uses counts recorded nodes that read this tensor
  cg::LazyNode* node = nullptr;
  int lazy_uses = 0;
  // a one-element literal keeps its value on the host (carried through views), so that chains such
  // as x / sqrt(mean + eps) can be recognised without reading device memory
  bool has_scalar = false;
  uint32_t scalar_bits = 0;

  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    return n;
  }
  bool contiguous() const {
    int64_t s = 1;
    for (int i = rank - 1; i >= 0; --i) {
      if (dims[i] != 1 && strides[i] != s) return false;
      s *= dims[i];
    }
    return true;
  }
  size_t esize() const { return cg::storage_bytes(storage); }
  void* data() const { return (char*)buf->ptr + (size_t)offset * esize(); }
};

namespace cg {

int fail(cg_ctx* c, int code, const std::string& msg);
int cuda_fail(cg_ctx* c, cudaError_t e, const char* what);

#define CG_CUDA(ctx, call)                                   \
  do {                                                       \
    cudaError_t e__ = (call);                                \
    if (e__ != cudaSuccess) return cg::cuda_fail(ctx, e__, #call); \
  } while (0)

// After a kernel launch: count it and surface launch errors.
#define CG_LAUNCHED(ctx)                                              \
  do {                                                                \
    (ctx)->launches++;                                                \
    cudaError_t e__ = cudaGetLastError();                             \
    if (e__ != cudaSuccess) return cg::cuda_fail(ctx, e__, "kernel launch"); \
  } while (0)

#define CG_TRY(expr)            \
  do {                          \
    int st__ = (expr);          \
    if (st__ != CG_OK) return st__; \
  } while (0)

// Function attributes (dynamic shared memory limit, cluster size) are set per device: call sites
// keep one of these per function so that every GPU a process uses gets configured once.
struct PerDeviceFlag {
  bool done[64] = {};
  bool& at(int device) { return done[device & 63]; }
};
struct PerDeviceSize {
  size_t v[64] = {};
  size_t& at(int device) { return v[device & 63]; }
};

// New contiguous tensor with fresh storage.
int new_tensor(cg_ctx* c, int tag, int storage, const int64_t* dims, int rank, cg_tensor** out);
// New handle sharing t's buffer (same view); caller edits dims/strides/offset.
cg_tensor* new_view(const cg_tensor* t);
void release(cg_tensor* t);

// RAII holder for temporaries inside entry points.
struct Hold {
  cg_tensor* t = nullptr;
  Hold() = default;
  explicit Hold(cg_tensor* p) : t(p) {}
  Hold(const Hold&) = delete;
  Hold& operator=(const Hold&) = delete;
  ~Hold() { if (t) release(t); }
  cg_tensor* take() { cg_tensor* p = t; t = nullptr; return p; }
};

// A contiguous tensor equal to x: x itself (retained) when already contiguous.
int as_contiguous(cg_ctx* c, const cg_tensor* x, cg_tensor** out);
// The [M, K] matrix that the last two axes of `a` (all leading axes folded into M; `a` must be
// contiguous over them, or rank 2) form, as a contiguous bf16 matrix: `a` itself when it is stored
// that way, else the rounded copy cached on its buffer (made on first use).  *keep holds whatever
// must stay alive while the pointer is used.
int bf16_operand(cg_ctx* c, const cg_tensor* a, int64_t M, int64_t K, int64_t row_stride, int64_t col_stride, cg_tensor** keep,
                 const __nv_bfloat16** out);
// Like as_contiguous but also widens bf16 storage to f32.
int as_contiguous_f32(cg_ctx* c, const cg_tensor* x, cg_tensor** out);

// Up to three operands sharing one iteration space, passed to kernels by value.
struct Iter {
  int rank;
  int64_t dims[CG_MAX_RANK];
  int64_t s0[CG_MAX_RANK], s1[CG_MAX_RANK], s2[CG_MAX_RANK];
};
// Build an Iter from shapes/strides, merging adjacent dims that are jointly contiguous
// in every operand and dropping unit dims.  Unused operands pass nullptr strides.
Iter make_iter(int rank, const int64_t* dims, const int64_t* s0, const int64_t* s1, const int64_t* s2);

// Launch on the context's stream with programmatic dependent launch (the kernel may start
// before its predecessor in the stream has finished; it must execute griddepcontrol.wait
// before it reads or writes anything the predecessor touches) and, when cluster_z > 1, as
// thread-block clusters of (1, 1, cluster_z); a negative cluster_z asks for clusters of
// (-cluster_z, 1, 1) instead (CTA pairs of tcgen05 cta_group::2 are neighbours along x).
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(cg_ctx* c, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_z,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->core->stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (c->opt_pdl) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1 || cluster_z < -1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_z < 0 ? (unsigned)-cluster_z : 1;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = cluster_z < 0 ? 1 : (unsigned)cluster_z;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

inline int grid_for(int64_t n, int block, int max_blocks = 148 * 16) {
  int64_t g = (n + block - 1) / block;
  if (g < 1) g = 1;
  if (g > max_blocks) g = max_blocks;
  return (int)g;
}

// ---- deferred evaluation (lazy.cu) ----------------------------------------------------
// Runs every recorded node (fused where a chain is recognised).  No-op when nothing is pending.
int lazy_flush(cg_ctx* c);
// Called when the last reference to a tensor that is still pending goes away.
void lazy_orphan(cg_tensor* t);
// Recorders: return true when the call was recorded (then *st is its status and *out the pending
// result); false when the caller should run eagerly.
bool lazy_binary(cg_ctx* c, int op, const cg_tensor* a, const cg_tensor* b, cg_tensor** out, int* st);
bool lazy_unary_neg(cg_ctx* c, const cg_tensor* x, cg_tensor** out, int* st);
bool lazy_reduce(cg_ctx* c, int red, const cg_tensor* x, cg_tensor** out, int* st);
bool lazy_cast(cg_ctx* c, const cg_tensor* x, int dtype, cg_tensor** out, int* st);
bool lazy_matmul(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out, int* st);
bool lazy_concat(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, int dim, cg_tensor** out, int* st);
bool lazy_arange(cg_ctx* c, int64_t end, cg_tensor** out, int* st);
// A view `t` of the pending tensor `x` was just created by metadata arithmetic: register it.
enum LazyView : int { LV_BROADCAST = 0, LV_TRANSPOSE = 1, LV_SLICE = 2, LV_RESHAPE = 3 };
void lazy_view(cg_ctx* c, int kind, cg_tensor* t, const cg_tensor* x, const int64_t* args, int nargs);
// reshape that needs a copy, of a pending tensor
int lazy_reshape_copy(cg_ctx* c, const cg_tensor* x, const int64_t* dims, int rank, cg_tensor** out);
enum LazyBin : int { LB_ADD = 0, LB_SUB, LB_MUL, LB_DIV, LB_POW, LB_LT };
enum LazyRed : int { LR_MAX = 0, LR_SUM };
// Run what is pending only if this tensor is part of it.
#define CG_LAZY_NEED(ctx, t)                                                                        \
  do {                                                                                              \
    if ((ctx) && (ctx)->lazy && !(ctx)->lazy_busy && (t) && (t)->node) CG_TRY(cg::lazy_flush(ctx)); \
  } while (0)
#define CG_LAZY_FLUSH(ctx)                                                  \
  do {                                                                      \
    if ((ctx) && (ctx)->lazy && !(ctx)->lazy_busy) CG_TRY(cg::lazy_flush(ctx)); \
  } while (0)

// Entry points outside the recorded trait methods (fused kernels, the decoder) first run whatever
// is pending and then execute eagerly, including the trait methods they call themselves.
struct LazyPause {
  cg_ctx* c;
  bool was;
  explicit LazyPause(cg_ctx* ctx) : c(ctx), was(ctx ? ctx->lazy_busy : false) { if (c) c->lazy_busy = true; }
  ~LazyPause() { if (c) c->lazy_busy = was; }
};
#define CG_LAZY_EAGER_SCOPE(ctx) \
  CG_LAZY_FLUSH(ctx);            \
  cg::LazyPause lazy_pause__(ctx)

// ---- entry points implemented in other translation units, used across them ----------

// y[M,N] = x[M,K] w[N,K]^T on the tcgen05 pipeline.  x, w bf16 row-major (ld in elements);
// out_mode 0: f32 store, 1: bf16 store, 2: f32 out = acc + residual (residual may alias out).
// splits <= 0 lets the launcher choose.  `workspace` must hold splits*M*N floats when
// splits > 1 (pass nullptr to have it allocated from the context).
int gemm_tc(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw,
            void* out, int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K,
            int out_mode, int splits, float* workspace);
// Persistent variant for many tokens (double-buffered TMEM accumulators, epilogue overlapped
// with the next tile's MMAs).  pair != 0: w holds N gate rows then N up rows (w_rows = 2 N) and
// out[M, N] (bf16) = act(x gate^T) * (x up^T).  gemm_tc and gemm_tc_pair route here by themselves
// when gemm_tcp_wanted says the problem is large enough.
bool gemm_tcp_wanted(int64_t M, int64_t N, int64_t K);
bool gemm_tcp2_supported(int64_t N, int glu);
bool gemm_tcp2_wanted(int64_t M, int64_t N, int64_t K, int glu);
int gemm_tcp2(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, int64_t w_rows, void* out,
              int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K, int out_mode, int glu, int act);
int gemm_tcp(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw, int64_t w_rows,
             void* out, int64_t ldo, const float* residual, int64_t M, int64_t N, int64_t K, int out_mode,
             int pair, int act);
int gemm_tcp_grouped(cg_ctx* c, const __nv_bfloat16* x, int64_t x_rows, const __nv_bfloat16* w, const __nv_bfloat16* w_up,
                     int64_t experts, void* out, int64_t N, int64_t K, int pair, int act, const int32_t* tile_expert,
                     const int32_t* tile_row0, const int32_t* tile_rows, const int32_t* n_list, int64_t max_list);
// Gate and up projections with the activation fused: w holds the gate rows then the up rows
// ([2 F, K]); out[M, F] (bf16) = act(x gate^T) * (x up^T), act 0 = silu, 1 = tanh-gelu.
int gemm_tc_pair(cg_ctx* c, const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, int64_t ldw,
                 __nv_bfloat16* out, int64_t ldo, int64_t M, int64_t F, int64_t K, int act);
// How many split-K slices gemm_tc would pick for this problem.
int gemm_tc_pick_splits(int64_t M, int64_t N, int64_t K);

// Generic strided f32 / u32 batched GEMM on CUDA cores (parity path).
int gemm_simt(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor* out);

}  // namespace cg
