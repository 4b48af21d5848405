// decode_resident.cu — all requested decode steps of a dense pre-norm decoder
// (catgrad-llm/src/models/llama.rs:117-151 per layer, the greedy loop of
// catgrad-llm/examples/llama/main.rs:118-169 around it) as ONE resident kernel.
//
// A decode step of a handful of rows streams every weight once and is otherwise a chain of ~80
// dependent small operations.  Run as one kernel per operation, each link of the chain pays
// a launch, a ramp-up and a drain during which HBM is idle.  Here one CTA per SM stays resident
// for the whole call and the chain is a sequence of PHASES separated by grid barriers:
//
//   per step:  embed | per layer: qkv GEMM, attention, o GEMM, gate/up GEMM, down GEMM | LM head
//
//   * The weight stream never stops at a phase boundary.  Which weight tile a CTA needs next is
//     known in advance (it depends on nothing computed), so warp 0 walks the whole schedule --
//     across phases, layers and steps -- issuing TMA loads into a shared-memory ring as slots
//     free up, without ever looking at a barrier.  While a CTA waits for a dependency, its ring
//     fills with the weights of the next GEMMs.
//   * Only the small activation tiles depend on the previous phase.  Warp 1 walks the same
//     schedule, waits for the grid barrier of the phase a tile belongs to, and then loads the
//     activation tile of each stage.
//   * Warp 2 issues tcgen05.mma (128 x TN x 16, f32 accumulators in TMEM, two accumulator
//     buffers so the next tile's MMAs overlap the previous tile's epilogue).
//   * Warps 4-7 are the epilogue of the GEMM phases and the workers of the other phases
//     (embedding, attention, greedy pick).
//   * CTAs form clusters of four.  A cluster owns whole 128-row weight tiles and its CTAs split
//     K four ways; partial tiles are summed in rank order over distributed shared memory, each
//     CTA finishing 32 of the 128 rows (deterministic: no atomics on floats anywhere).
//   * The RMSNorms ride on the GEMMs as in gemm_dec.cu: a residual GEMM also leaves
//     bf16(x * gain) and per-CTA sums of squares, the GEMM behind the norm scales its
//     accumulator rows by 1 / rms.
//   * Attention is attn_decode.cuh's item function; the slices of one (row, kv head) are held by
//     CTAs of one cluster and merged over distributed shared memory.
//
// Barriers between CTAs are mbarriers (inside a cluster) and one monotonically increasing
// counter in global memory (grid wide).  Every wait is bounded: when a limit runs out the CTA
// raises the context's error word, every role leaves its loop, copies still in flight are
// waited for, TMEM is freed and the kernel returns; later waits of other CTAs give up as soon
// as they see the word.  All CTAs must be co-resident: the grid is sized from the occupancy
// query and the kernel takes a whole SM's shared memory, so nothing else shares an SM with it.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

#include "act.cuh"
#include "attn_decode.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace cg {

namespace {

using namespace tc;

constexpr int R_THREADS = 256;
constexpr int R_CS = 4;            // CTAs per cluster = K slices per weight tile
constexpr int R_ROWS = BM / R_CS;  // rows of a tile each CTA finishes (one per lane)
constexpr int EPI0 = 128;          // first worker thread (warps 4-7)
constexpr int R_MAX_STAGES = 12;
constexpr int R_ACC_COLS = 128;    // TMEM columns: two buffers of 64

enum : int { PH_EMBED = 0, PH_GEMM = 1, PH_ATTN = 2 };
enum : int { EP_SCALE_F32 = 0, EP_RESIDUAL = 1, EP_ACTMUL = 2, EP_HEAD = 3 };

struct RPhase {
  int kind, layer;
  int map_w, map_x;
  int n_tiles, kb_total, dual, up_off;
  int epi, N, ldo, rot;
  int ss_parts_in, ss_slot_in, ss_slot_out, pad;
  void* out;          // EP_SCALE_F32 / EP_HEAD: f32 [M, ldo]; EP_ACTMUL: bf16 [M, ldo]
  const float* gain;  // EP_RESIDUAL: gain of the norm that follows
};

struct RLayer {
  __nv_bfloat16 *k_cache, *v_cache;
  const float *q_gamma, *k_gamma, *cos_t, *sin_t;
  int64_t window;
};

struct RArgs {
  const RPhase* phases;
  const RLayer* layers;
  const CUtensorMap* maps;
  int n_phases, n_steps, n_clusters, stages, gen_bytes, attn_group;
  int M, H, nh, nkv, d, qkv_ld, Tmax, vocab, act, plus_one, embed_storage;
  float eps, attn_scale, attn_softcap, final_softcap, embed_scale;
  float* x;               // [M, H] f32 residual stream
  __nv_bfloat16* xn;      // [M, H] bf16(x * gain), un-normalised
  float* ss;              // [2][parts][32] partial sums of squares
  int64_t ss_stride;      // floats per ss slot
  const float* qkv;       // [M, qkv_ld] f32 (written by the qkv GEMM)
  __nv_bfloat16* att;     // [M, nh d]
  const void* embed;
  const float* gain0;     // first layer's input norm gain
  uint32_t* cur;          // [M] tokens the first step consumes; the last step's pick on return
  uint32_t* history;
  int64_t hist_ld;
  int64_t* count_dev;
  int64_t* pos_dev;
  unsigned long long* best;  // [M] zeroed merge slots of the greedy pick
  unsigned* bar;          // grid barrier counter, zero at launch
  int32_t* err;
  // diagnostics: CTA `trace_cta` stamps globaltimer when each of the first trace_cap phases may
  // start (its grid barrier passed) and when this CTA has finished its part of the phase
  unsigned long long* trace;
  int trace_cap, trace_cta;
  int prefetch_ahead;  // stages the L2 prefetcher may run ahead of the weight producer (0 = no prefetch)
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait until the grid barrier counter reaches `target`.
__device__ __forceinline__ bool grid_wait(const unsigned* bar, unsigned target, volatile int* cta_abort, int32_t* err) {
  uint64_t t0 = 0, limit = 0;
  for (uint32_t it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
    if ((int)(v - target) >= 0) return true;
    if ((it & 0xFF) == 0xFF) {
      if (*cta_abort) return false;
      if (*(volatile int32_t*)err == DEV_TIMEOUT) break;
      uint64_t now = globaltimer();
      if (t0 == 0) { t0 = now; limit = wait_limit_ns(err); }
      else if (now - t0 > limit) break;
    }
  }
  *cta_abort = 1;
  *err = DEV_TIMEOUT;
  return false;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ float sum4_cluster_f32(uint32_t local_addr) {
  float v[R_CS];
#pragma unroll
  for (int s = 0; s < R_CS; ++s) v[s] = ld_cluster_f32(local_addr, (uint32_t)s);
  return ((v[0] + v[1]) + v[2]) + v[3];
}
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t index) {
  const uint32_t bits = __float_as_uint(v);
  const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // f32::total_cmp order
  return ((unsigned long long)key << 32) | index;                           // ties -> last index
}

// tcgen05.mma with the accumulate flag fixed at compile time (no predicate arithmetic per issue)
__device__ __forceinline__ void umma_bf16_first(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_acc(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc)
      : "memory");
}
// Position in the shared-memory ring: slot index and the parity of the slot's current use.  The
// roles advance it once per stage (no division by the runtime ring depth on the issue path).
struct RingPos {
  uint32_t s = 0, par = 0, round = 0;
  __device__ __forceinline__ void advance(uint32_t nst) {
    if (++s == nst) { s = 0; par ^= 1u; round = 1; }
  }
};

// The walk every role makes over the static schedule: steps, phases, this cluster's tiles of a
// GEMM phase, this CTA's k blocks, and (gate/up pairs) the two weight tiles of a k block.
struct Walk {
  const RArgs& p;
  int cl, rank;
  __device__ Walk(const RArgs& a, int cluster, int r) : p(a), cl(cluster), rank(r) {}
  __device__ __forceinline__ int first_tile(const RPhase& ph) const {
    int t = (cl - ph.rot) % p.n_clusters;
    return t < 0 ? t + p.n_clusters : t;
  }
  __device__ __forceinline__ int kb0(const RPhase& ph) const { return rank * ph.kb_total / R_CS; }
  __device__ __forceinline__ int kb1(const RPhase& ph) const { return (rank + 1) * ph.kb_total / R_CS; }
};

// Environment of attn_dec_item inside the resident kernel: 128 worker threads, the slices of a
// (row, kv head) on `group` consecutive CTAs of the cluster, a group barrier made of mbarriers.
struct ResidentAttnEnv {
  uint32_t gbar;        // this CTA's group barrier (count = group size)
  uint32_t phase;       // parity of the next completion
  int group, base;      // group size, cluster rank of the group's first CTA
  volatile int* cta_abort;
  int32_t* err;
  __device__ __forceinline__ int tid() const { return (int)threadIdx.x - EPI0; }
  __device__ __forceinline__ void sync_cta() const { epi_sync(); }
  __device__ __forceinline__ void sync_group() {
    epi_sync();
    if (group == 1) return;
    const int t = tid();
    if (t < group) mbar_arrive_remote(gbar, (uint32_t)(base + t));
    mbar_wait_cluster(gbar, phase, cta_abort, err);
    phase ^= 1u;
  }
  __device__ __forceinline__ uint32_t cluster_rank(int s) const { return (uint32_t)(base + s); }
  __device__ __forceinline__ int64_t settle(int64_t pos) const { return pos; }  // the phase barrier came first
  // items follow one another in a CTA: partials are read where they lie, behind two barriers
  static constexpr bool kPush = false;
  __device__ __forceinline__ float* landing() const { return nullptr; }
};

template <int TN, int D>
__global__ void __launch_bounds__(R_THREADS, 1) k_decode_resident(const __grid_constant__ RArgs p) {
  constexpr uint32_t X_TILE = TN * BK * 2;
  constexpr uint32_t STAGE = A_BYTES + X_TILE;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen0 = smem_raw + (base - raw);
  const int NST = p.stages;
  const uint32_t ring = base;
  const uint32_t gen = base + (uint32_t)NST * STAGE;           // staging of the cluster reduction / attention scratch
  uint8_t* gen_ptr = gen0 + (size_t)NST * STAGE;
  const uint32_t bars = gen + (uint32_t)p.gen_bytes;
  uint8_t* bars_ptr = gen_ptr + p.gen_bytes;
  // barriers: full[NST], empty[NST], acc_full[2], acc_empty[2], cbar, gbar
  const uint32_t b_full = bars, b_empty = bars + 8 * R_MAX_STAGES, b_accf = bars + 16 * R_MAX_STAGES,
                 b_acce = b_accf + 16, b_cbar = b_acce + 16, b_gbar = b_cbar + 8;
  uint8_t* misc = bars_ptr + 16 * R_MAX_STAGES + 64;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)misc;
  volatile int* cta_abort = (volatile int*)(misc + 4);
  volatile int* w_issued = (volatile int*)(misc + 8);
  volatile int* x_issued = (volatile int*)(misc + 12);
  volatile int* consumed = (volatile int*)(misc + 16);
  volatile int* w_pos = (volatile int*)(misc + 20);   // stages the weight producer has issued so far (read by the prefetcher)
  float* sc = (float*)(misc + 32);        // [32] per-row 1 / rms of the phase
  float* red = (float*)(misc + 32 + 128); // [8] block reductions of the workers

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = (int)cluster_ctarank();
  const int cl = blockIdx.x / R_CS;
  const unsigned n_ctas = gridDim.x;
  Walk walk(p, cl, rank);

  if (tid == 0) {
    for (int s = 0; s < R_MAX_STAGES; ++s) {
      mbar_init(b_full + 8 * s, 2);   // weight arrival + activation arrival
      mbar_init(b_empty + 8 * s, 1);  // one tcgen05.commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_accf + 8 * s, 1);   // one tcgen05.commit
      mbar_init(b_acce + 8 * s, 4);   // one arrival per worker warp
    }
    mbar_init(b_cbar, R_CS);
    mbar_init(b_gbar, (uint32_t)p.attn_group);
    *cta_abort = 0;
    *w_issued = 0;
    *x_issued = 0;
    *consumed = 0;
    *w_pos = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"((uint32_t)R_ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // every CTA's barriers exist before any remote arrive
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  // counters at kernel entry; written back by the last phase
  const int64_t count0 = *p.count_dev, pos0 = *p.pos_dev;

  if (warp == 0) {
    // ---------------- weight producer: free-running over the whole schedule ----------------
    if (lane == 0) {
      int st = 0;
      RingPos rp;
      bool ok = true;
      for (int step = 0; step < p.n_steps && ok; ++step) {
        for (int pi = 0; pi < p.n_phases && ok; ++pi) {
          const RPhase ph = p.phases[pi];  // by value: the fields stay in registers across the asm statements
          if (ph.kind != PH_GEMM) continue;
          const CUtensorMap* mw = p.maps + ph.map_w;
          const int k0 = walk.kb0(ph), k1 = walk.kb1(ph);
          for (int t = walk.first_tile(ph); t < ph.n_tiles && ok; t += p.n_clusters) {
            for (int kb = k0; kb < k1 && ok; ++kb) {
              for (int h = 0; h <= ph.dual; ++h, ++st) {
                // (a slot's first use needs no wait; later uses wait for the MMAs that read it)
                if (rp.round && !mbar_wait(b_empty + 8 * rp.s, rp.par ^ 1u, cta_abort, p.err)) { ok = false; break; }
                mbar_expect_tx(b_full + 8 * rp.s, A_BYTES);
                tma_load_2d(ring + rp.s * STAGE, mw, kb * BK, t * BM + h * ph.up_off, b_full + 8 * rp.s);
                rp.advance((uint32_t)NST);
                *w_pos = st + 1;
              }
            }
          }
        }
      }
      *w_issued = st;
    }
  } else if (warp == 1) {
    // ---------------- activation producer: same walk, gated by the grid barrier ----------------
    if (lane == 0) {
      int st = 0;
      RingPos rp;
      bool ok = true;
      for (int step = 0; step < p.n_steps && ok; ++step) {
        for (int pi = 0; pi < p.n_phases && ok; ++pi) {
          const RPhase ph = p.phases[pi];  // by value: the fields stay in registers across the asm statements
          if (ph.kind != PH_GEMM) continue;
          const int t0 = walk.first_tile(ph);
          if (t0 >= ph.n_tiles) continue;
          // the phase's inputs are complete once every CTA has arrived for all earlier phases
          const unsigned g = (unsigned)(step * p.n_phases + pi);
          if (!grid_wait(p.bar, g * n_ctas, cta_abort, p.err)) { ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");  // other CTAs' generic-proxy stores before the TMA reads
          const CUtensorMap* mx = p.maps + ph.map_x;
          const int k0 = walk.kb0(ph), k1 = walk.kb1(ph);
          for (int t = t0; t < ph.n_tiles && ok; t += p.n_clusters) {
            for (int kb = k0; kb < k1 && ok; ++kb) {
              for (int h = 0; h <= ph.dual; ++h, ++st) {
                if (rp.round && !mbar_wait(b_empty + 8 * rp.s, rp.par ^ 1u, cta_abort, p.err)) { ok = false; break; }
                mbar_expect_tx(b_full + 8 * rp.s, X_TILE);
                tma_load_2d(ring + rp.s * STAGE + A_BYTES, mx, kb * BK, 0, b_full + 8 * rp.s);
                rp.advance((uint32_t)NST);
              }
            }
          }
        }
      }
      *x_issued = st;
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(TN);
      // descriptors of slot 0; a slot further on adds its byte offset / 16 to the address field
      const uint64_t desc_a0 = umma_desc(ring), desc_b0 = umma_desc(ring + A_BYTES);
      int st = 0, u = 0;
      RingPos rp;
      bool ok = true;
      for (int step = 0; step < p.n_steps && ok; ++step) {
        for (int pi = 0; pi < p.n_phases && ok; ++pi) {
          const RPhase ph = p.phases[pi];  // by value: the fields stay in registers across the asm statements
          if (ph.kind != PH_GEMM) continue;
          const int k0 = walk.kb0(ph), k1 = walk.kb1(ph);
          for (int t = walk.first_tile(ph); t < ph.n_tiles && ok; t += p.n_clusters, ++u) {
            const int buf = u & 1;
            // the workers have read this buffer's previous tile
            if (!mbar_wait(b_acce + 8 * buf, ((uint32_t)(u >> 1) & 1u) ^ 1u, cta_abort, p.err)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_acc + (uint32_t)(buf * 64);
            for (int kb = k0; kb < k1 && ok; ++kb) {
              for (int h = 0; h <= ph.dual; ++h, ++st) {
                if (!mbar_wait(b_full + 8 * rp.s, rp.par, cta_abort, p.err)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t off = (uint64_t)(rp.s * (STAGE >> 4));
                const uint64_t da = desc_a0 + off, db = desc_b0 + off;
                const uint32_t d = acc + (uint32_t)(h * TN);
                if (kb == k0) umma_bf16_first(d, da, db, idesc);
                else umma_bf16_acc(d, da, db, idesc);
#pragma unroll
                for (int kk = 1; kk < BK / UMMA_K; ++kk)
                  umma_bf16_acc(d, da + (uint64_t)(kk * (UMMA_K * 2 >> 4)), db + (uint64_t)(kk * (UMMA_K * 2 >> 4)), idesc);
                umma_commit(b_empty + 8 * rp.s);
                rp.advance((uint32_t)NST);
              }
            }
            if (ok) umma_commit(b_accf + 8 * buf);
          }
        }
      }
      *consumed = st;
    }
  } else if (warp == 3) {
    // ---------------- L2 prefetcher: the same walk, a bounded distance ahead of the weight producer ----------------
    // A CTA's ring holds a few microseconds of weights; when the dependency chain stalls for longer
    // the ring is full and this SM would stop pulling from HBM.  Prefetches into L2 return nothing to
    // the SM, so they keep HBM busy meanwhile, and the ring later refills at L2 latency.
    if (lane == 0 && p.prefetch_ahead > 0) {
      int st = 0;
      bool ok = true;
      for (int step = 0; step < p.n_steps && ok; ++step) {
        for (int pi = 0; pi < p.n_phases && ok; ++pi) {
          const RPhase ph = p.phases[pi];
          if (ph.kind != PH_GEMM) continue;
          const CUtensorMap* mw = p.maps + ph.map_w;
          const int k0 = walk.kb0(ph), k1 = walk.kb1(ph);
          for (int t = walk.first_tile(ph); t < ph.n_tiles && ok; t += p.n_clusters) {
            for (int kb = k0; kb < k1 && ok; ++kb) {
              for (int h = 0; h <= ph.dual; ++h, ++st) {
                // stay within prefetch_ahead stages of what the producer has issued
                uint32_t spins = 0;
                while (st - *w_pos >= p.prefetch_ahead) {
                  __nanosleep(100);
                  if ((++spins & 0x3FF) == 0 && (*cta_abort || *(volatile int32_t*)p.err == DEV_TIMEOUT)) { ok = false; break; }
                }
                if (!ok) break;
                if (st >= *w_pos)  // (already loaded stages need no prefetch)
                  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(mw), "r"(kb * BK),
                               "r"(t * BM + h * ph.up_off)
                               : "memory");
              }
            }
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ---------------- workers: epilogues, embedding, attention, greedy pick ----------------
    const int et = tid - EPI0, ew = et >> 5;  // worker thread / warp index; ew = TMEM lane quarter
    float* stage = (float*)gen_ptr;           // [2 buffers][2 TN columns][128 rows]
    uint32_t cph = 0;                         // parity of the cluster barrier's next completion
    ResidentAttnEnv env;
    env.gbar = b_gbar; env.phase = 0; env.group = p.attn_group; env.base = rank / p.attn_group * p.attn_group;
    env.cta_abort = cta_abort; env.err = p.err;
    int u = 0;
    bool ok = true;
    const int total_phases = p.n_steps * p.n_phases;
    for (int gph = 0; gph <= total_phases && ok; ++gph) {
      const int step = gph / p.n_phases, pi = gph - step * p.n_phases;
      // every CTA has finished all earlier phases (and this CTA may now arrive for this one)
      if (et == 0) {
        if (!grid_wait(p.bar, (unsigned)gph * n_ctas, cta_abort, p.err)) *cta_abort = 1;
        __threadfence();
      }
      epi_sync();
      if (*cta_abort) { ok = false; break; }
      if (et == 0 && p.trace && (int)blockIdx.x == p.trace_cta && gph < p.trace_cap) p.trace[2 * gph] = globaltimer();
      const bool final_phase = gph == total_phases;
      const RPhase ph = p.phases[final_phase ? 0 : pi];
      if (ph.kind == PH_EMBED) {
        // the greedy pick of the previous step (or the tokens handed in), then the next step's
        // embedding rows with the first norm's hand-over
        for (int m = blockIdx.x; m < p.M; m += (int)n_ctas) {
          uint32_t tok;
          if (step == 0) {
            tok = __ldcg(p.cur + m);
          } else {
            tok = (uint32_t)(__ldcg(p.best + m) & 0xFFFFFFFFull);
            epi_sync();  // everyone has read the slot
            if (et == 0) {
              p.best[m] = 0ull;
              p.cur[m] = tok;
              if (p.history) p.history[(int64_t)m * p.hist_ld + count0 + step - 1] = tok;
            }
          }
          if (final_phase) continue;
          if (tok >= (uint32_t)p.vocab) { if (et == 0) *p.err = DEV_INDEX; tok = 0; }
          float sq = 0.f;
          if (p.embed_storage == ST_BF16) {
            // eight elements per thread and pass: 16-byte loads of the table row, 16-byte stores
            const uint4* trow = (const uint4*)((const __nv_bfloat16*)p.embed + (int64_t)tok * p.H);
            for (int i = et; i < p.H / 8; i += 128) {
              const uint4 raw4 = trow[i];
              const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw4;
              const float4 ga = ((const float4*)p.gain0)[2 * i], gb = ((const float4*)p.gain0)[2 * i + 1];
              const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
              float v[8];
              __nv_bfloat162 o2[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h2[j]);
                v[2 * j] = f.x * p.embed_scale;
                v[2 * j + 1] = f.y * p.embed_scale;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) sq += v[j] * v[j];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                o2[j] = __floats2bfloat162_rn(v[2 * j] * (p.plus_one ? 1.f + gg[2 * j] : gg[2 * j]),
                                              v[2 * j + 1] * (p.plus_one ? 1.f + gg[2 * j + 1] : gg[2 * j + 1]));
              float4* xo = (float4*)(p.x + (int64_t)m * p.H) + 2 * i;
              xo[0] = make_float4(v[0], v[1], v[2], v[3]);
              xo[1] = make_float4(v[4], v[5], v[6], v[7]);
              ((uint4*)(p.xn + (int64_t)m * p.H))[i] = *(const uint4*)o2;
            }
          } else {
            for (int i = et; i < p.H; i += 128) {
              const float v = ((const float*)p.embed)[(int64_t)tok * p.H + i] * p.embed_scale;
              p.x[(int64_t)m * p.H + i] = v;
              const float g = p.plus_one ? 1.f + p.gain0[i] : p.gain0[i];
              p.xn[(int64_t)m * p.H + i] = __float2bfloat16_rn(v * g);
              sq += v * v;
            }
          }
#pragma unroll
          for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (lane == 0) red[ew] = sq;
          epi_sync();
          if (et == 0) p.ss[(int64_t)ph.ss_slot_out * p.ss_stride + m] = ((red[0] + red[1]) + red[2]) + red[3];
          epi_sync();
        }
        if (final_phase) {
          if (blockIdx.x == 0 && et == 0) {
            *p.count_dev = count0 + p.n_steps;
            *p.pos_dev = pos0 + p.n_steps;
          }
          break;  // nothing follows: no arrival needed
        }
      } else if (ph.kind == PH_ATTN) {
        const RLayer& L = p.layers[ph.layer];
        AttnDecArgs a;
        a.qkv = p.qkv; a.cos_t = L.cos_t; a.sin_t = L.sin_t; a.q_gamma = L.q_gamma; a.k_gamma = L.k_gamma;
        a.norm_eps = p.eps; a.norm_plus_one = p.plus_one; a.k_cache = L.k_cache; a.v_cache = L.v_cache; a.out = p.att;
        a.pos_dev = nullptr; a.pos0 = pos0 + step; a.Tmax = p.Tmax; a.B = p.M; a.nh = p.nh; a.nkv = p.nkv; a.d = D;
        a.window = L.window; a.softcap = p.attn_softcap; a.splits = p.attn_group; a.push_merge = 0;
        const int groups_per_cluster = R_CS / p.attn_group;
        const int n_groups = p.n_clusters * groups_per_cluster;
        const int pairs = p.M * p.nkv;
        for (int pr = cl * groups_per_cluster + rank / p.attn_group; pr < pairs && !*cta_abort; pr += n_groups) {
          attn_dec_item<D>(a, p.attn_scale, pr % p.nkv, (int64_t)(pr / p.nkv), rank % p.attn_group, pos0 + step, gen_ptr, env);
          // (the item ends with a group barrier or a worker barrier: its scratch is free again)
        }
      } else {
        // ---- GEMM phase: this cluster's tiles ----
        if (ph.ss_parts_in > 0) {
          // per-row 1 / rms from the producer's partial sums, added in a fixed order
          const int m = et >> 2, j = et & 3;
          const float* ssin = p.ss + (int64_t)ph.ss_slot_in * p.ss_stride;
          float a = 0.f;
          if (m < p.M)
            for (int i = j; i < ph.ss_parts_in; i += 4) a += __ldcg(ssin + (int64_t)i * 32 + m);
          const float a1 = __shfl_down_sync(0xffffffffu, a, 1), a2 = __shfl_down_sync(0xffffffffu, a, 2),
                      a3 = __shfl_down_sync(0xffffffffu, a, 3);
          if (j == 0 && m < p.M) sc[m] = 1.0f / sqrtf((((a + a1) + a2) + a3) / (float)(ph.kb_total * BK) + p.eps);
          epi_sync();
        }
        unsigned long long hb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) hb[i] = 0ull;
        float* ss_out = ph.epi == EP_RESIDUAL ? p.ss + (int64_t)ph.ss_slot_out * p.ss_stride : nullptr;
        for (int t = walk.first_tile(ph); t < ph.n_tiles && ok; t += p.n_clusters, ++u) {
          const int buf = u & 1;
          // this CTA finishes rows [rank * 32, rank * 32 + 32) of the tile: lane = row, worker warp
          // ew takes columns (rows of the batch) ew, ew + 4, ...  What the epilogue reads from
          // global memory is requested before the accumulator is waited for.
          const int frow = rank * R_ROWS + lane;
          const int n = t * BM + frow;
          const bool n_in = n < ph.N;
          float xres[8], gn = 0.f;
          if (ph.epi == EP_RESIDUAL && n_in) {
#pragma unroll
            for (int slot = 0; slot < 8; ++slot) {
              const int col = ew + 4 * slot;
              xres[slot] = col < p.M ? __ldcg(p.x + (int64_t)col * ph.ldo + n) : 0.f;
            }
            gn = p.plus_one ? 1.f + ph.gain[n] : ph.gain[n];
          }
          if (!mbar_wait(b_accf + 8 * buf, (uint32_t)(u >> 1) & 1u, cta_abort, p.err)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          float* sb = stage + (size_t)buf * 2 * TN * BM;
          const int row = ew * 32 + lane;
#pragma unroll 1
          for (int c0 = 0; c0 < TN; c0 += 16) {
            if (c0 >= p.M) break;
            uint32_t g[16], uu[16];
            tmem_ld16(tmem_acc + (uint32_t)(buf * 64) + ((uint32_t)(ew * 32) << 16) + (uint32_t)c0, g);
            if (ph.dual) tmem_ld16(tmem_acc + (uint32_t)(buf * 64) + ((uint32_t)(ew * 32) << 16) + (uint32_t)(TN + c0), uu);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              sb[(c0 + j) * BM + row] = __uint_as_float(g[j]);
              if (ph.dual) sb[(TN + c0 + j) * BM + row] = __uint_as_float(uu[j]);
            }
          }
          // the accumulator buffer is free for the tile after next
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(b_acce + 8 * buf);
          // all four partial tiles of the cluster are staged
          epi_sync();
          if (et < R_CS) mbar_arrive_remote(b_cbar, (uint32_t)et);
          if (!mbar_wait_cluster(b_cbar, cph, cta_abort, p.err)) { ok = false; break; }
          cph ^= 1u;
          const uint32_t sb_u = gen + (uint32_t)((size_t)buf * 2 * TN * BM * 4);
#pragma unroll
          for (int slot = 0; slot < 8; ++slot) {
            const int col = ew + 4 * slot;
            if (col >= p.M) break;
            float g = sum4_cluster_f32(sb_u + (uint32_t)(col * BM + frow) * 4u);
            float r2 = 0.f;
            if (n_in) {
              const int64_t o = (int64_t)col * ph.ldo + n;
              if (ph.epi == EP_RESIDUAL) {
                const float r = g + xres[slot];
                p.x[o] = r;
                p.xn[o] = __float2bfloat16_rn(r * gn);
                r2 = r * r;
              } else if (ph.epi == EP_ACTMUL) {
                float uv = sum4_cluster_f32(sb_u + (uint32_t)((TN + col) * BM + frow) * 4u);
                g *= sc[col];
                uv *= sc[col];
                ((__nv_bfloat16*)ph.out)[o] = __float2bfloat16_rn((p.act == 0 ? silu_f(g) : gelu_f(g)) * uv);
              } else {
                if (ph.ss_parts_in > 0) g *= sc[col];
                if (ph.epi == EP_HEAD) {
                  if (p.final_softcap > 0.f) g = p.final_softcap * tanh_f(g / p.final_softcap);
                  const unsigned long long q = argmax_key(g, (uint32_t)n);
                  hb[slot] = q > hb[slot] ? q : hb[slot];
                }
                ((float*)ph.out)[o] = g;
              }
            }
            if (ss_out) {
#pragma unroll
              for (int o2 = 16; o2; o2 >>= 1) r2 += __shfl_xor_sync(0xffffffffu, r2, o2);
              if (lane == 0) ss_out[((int64_t)t * R_CS + rank) * 32 + col] = r2;
            }
          }
        }
        if (ph.epi == EP_HEAD) {
#pragma unroll
          for (int slot = 0; slot < 8; ++slot) {
            const int col = ew + 4 * slot;
            if (col >= p.M) break;
            unsigned long long q = hb[slot];
#pragma unroll
            for (int o2 = 16; o2; o2 >>= 1) {
              const unsigned long long w = __shfl_xor_sync(0xffffffffu, q, o2);
              q = w > q ? w : q;
            }
            if (lane == 0 && q) atomicMax(p.best + col, q);
          }
        }
      }
      if (!ok) break;
      // this CTA's part of the phase is done: publish it and arrive
      if (et == 0 && p.trace && (int)blockIdx.x == p.trace_cta && gph < p.trace_cap) p.trace[2 * gph + 1] = globaltimer();
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      epi_sync();
      if (et == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar) : "memory");
    }
  }

  // ---------------- teardown ----------------
  __syncthreads();
  if (warp == 2 && lane == 0) {
    // after an abort some copies may still be in flight: complete their barriers and wait for them
    const int wi = *w_issued, xi = *x_issued, hi = wi > xi ? wi : xi;
    for (int i = *consumed; i < hi; ++i) {
      const int s = i % NST;
      if (i >= wi) mbar_arrive(b_full + 8 * s);
      if (i >= xi) mbar_arrive(b_full + 8 * s);
      uint32_t done = 0;
      for (int it = 0; it < (1 << 22) && !done; ++it)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(b_full + 8 * s), "r"((uint32_t)(i / NST) & 1u)
            : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // nobody leaves while a peer may still read its shared memory or arrive on its barriers
  if (warp == 2) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)R_ACC_COLS) : "memory");
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// host side

struct ResidentPlan {
  RArgs args{};
  int tn = 16, d = 64;
  size_t smem = 0;
  int grid = 0;
  void* dev_blob = nullptr;  // phases, layers, tensor maps, barrier counter
  size_t blob_bytes = 0;
  unsigned long long* trace_area = nullptr;
  std::shared_ptr<Core> core;
  int64_t algorithmic_bytes = 0;
};

namespace {

template <int TN, int D>
int configure(cg_ctx* c, size_t smem, int* max_clusters) {
  static PerDeviceSize configured_on;
  size_t& configured = configured_on.at(c->core->device);
  if (smem > configured) {
    CG_CUDA(c, cudaFuncSetAttribute(k_decode_resident<TN, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(R_CS * 64);
  cfg.blockDim = dim3(R_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = R_CS; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  int n = 0;
  CG_CUDA(c, cudaOccupancyMaxActiveClusters(&n, k_decode_resident<TN, D>, &cfg));
  *max_clusters = n;
  return CG_OK;
}

template <int TN, int D>
int launch(cg_ctx* c, const ResidentPlan& pl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.grid);
  cfg.blockDim = dim3(R_THREADS);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = c->core->stream;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = R_CS; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  CG_CUDA(c, cudaLaunchKernelEx(&cfg, k_decode_resident<TN, D>, pl.args));
  CG_LAUNCHED(c);
  return CG_OK;
}

template <int TN, int D>
size_t gen_bytes_of() {
  const size_t staging = (size_t)2 * 2 * TN * BM * 4;
  const size_t attn = attn_dec_smem_bytes<D>();
  return (std::max(staging, attn) + 1023) / 1024 * 1024;
}

}  // namespace

bool decode_resident_supported(const ResidentModel& m, int64_t M) {
  if (M < 1 || M > 32) return false;
  if (m.d != 64 && m.d != 128) return false;
  if (m.nkv <= 0 || m.nh % m.nkv || m.nh / m.nkv > ATTN_MAX_REP) return false;
  if (m.H % BK || m.F % BK || (m.nh * m.d) % BK) return false;
  if (m.H / BK < R_CS || m.F / BK < R_CS || (m.nh * m.d) / BK < R_CS) return false;
  if ((int64_t)(m.H / BM + 1) * R_CS > m.ss_parts_cap / 2) return false;
  return !m.layers.empty();
}

int decode_resident_prepare(cg_ctx* c, const ResidentModel& m, int64_t M, ResidentPlan** out) {
  *out = nullptr;
  if (!decode_resident_supported(m, M)) return fail(c, CG_ERR_UNSUPPORTED, "resident decode: unsupported shape");
  auto pl = std::unique_ptr<ResidentPlan>(new ResidentPlan());
  pl->core = c->core;
  pl->tn = M <= 16 ? 16 : 32;
  pl->d = m.d;
  const size_t gen = pl->tn == 16 ? (m.d == 64 ? gen_bytes_of<16, 64>() : gen_bytes_of<16, 128>())
                                  : (m.d == 64 ? gen_bytes_of<32, 64>() : gen_bytes_of<32, 128>());
  const size_t stage = A_BYTES + (size_t)pl->tn * BK * 2;
  const size_t fixed = 1024 + gen + 16 * R_MAX_STAGES + 64 + 32 + 128 + 64;
  const size_t budget = 227 * 1024;
  int stages = (int)((budget - fixed) / stage);
  stages = std::min(stages, R_MAX_STAGES);
  if (c->opt_res_stages >= 3) stages = std::min(stages, c->opt_res_stages);
  if (stages < 3) return fail(c, CG_ERR_UNSUPPORTED, "resident decode: not enough shared memory for the ring");
  pl->smem = fixed + (size_t)stages * stage;
  int max_clusters = 0;
  if (pl->tn == 16 && m.d == 64) CG_TRY((configure<16, 64>(c, pl->smem, &max_clusters)));
  else if (pl->tn == 16) CG_TRY((configure<16, 128>(c, pl->smem, &max_clusters)));
  else if (m.d == 64) CG_TRY((configure<32, 64>(c, pl->smem, &max_clusters)));
  else CG_TRY((configure<32, 128>(c, pl->smem, &max_clusters)));
  if (max_clusters < 8) return fail(c, CG_ERR_UNSUPPORTED, "resident decode: too few co-resident clusters on this device");
  const int NC = max_clusters;
  pl->grid = NC * R_CS;

  // ---- the static schedule of one step ----
  const int L = (int)m.layers.size();
  std::vector<RPhase> phases;
  std::vector<RLayer> layers(L);
  std::vector<CUtensorMap> maps;
  auto add_map = [&](const void* ptr, int64_t rows, int64_t cols, int box_rows, int* idx) -> int {
    CUtensorMap mp;
    CG_TRY(make_map(c, &mp, ptr, rows, cols, cols, box_rows));
    *idx = (int)maps.size();
    maps.push_back(mp);
    return CG_OK;
  };
  int mx_xn = 0, mx_att = 0, mx_h = 0;
  CG_TRY(add_map(m.xn, M, m.H, pl->tn, &mx_xn));
  CG_TRY(add_map(m.att, M, (int64_t)m.nh * m.d, pl->tn, &mx_att));
  CG_TRY(add_map(m.hact, M, m.F, pl->tn, &mx_h));
  int cursor = 0;  // round-robin position: consecutive phases continue where the last one stopped
  int64_t bytes = 0;
  auto gemm_phase = [&](const __nv_bfloat16* w, int64_t rows, int64_t K, int64_t N, int dual, int mapx, int epi, void* outp,
                        int64_t ldo, const float* gain, int parts_in, int slot_in, int slot_out, int layer) -> int {
    RPhase ph{};
    ph.kind = PH_GEMM; ph.layer = layer;
    CG_TRY(add_map(w, rows, K, BM, &ph.map_w));
    ph.map_x = mapx;
    ph.n_tiles = (int)((N + BM - 1) / BM);
    ph.kb_total = (int)(K / BK);
    ph.dual = dual; ph.up_off = dual ? (int)N : 0;
    ph.epi = epi; ph.N = (int)N; ph.ldo = (int)ldo; ph.rot = cursor;
    ph.ss_parts_in = parts_in; ph.ss_slot_in = slot_in; ph.ss_slot_out = slot_out;
    ph.out = outp; ph.gain = gain;
    cursor = (cursor + ph.n_tiles) % NC;
    bytes += rows * K * 2;
    phases.push_back(ph);
    return CG_OK;
  };
  {
    RPhase e{};
    e.kind = PH_EMBED; e.ss_slot_out = 0;
    phases.push_back(e);
  }
  const int parts_res = (int)(m.H / BM + (m.H % BM ? 1 : 0)) * R_CS;  // partial sums a residual GEMM writes
  int parts = 1, slot = 0;  // the embedding writes one partial per row into slot 0
  for (int li = 0; li < L; ++li) {
    const ResidentLayerDesc& Ld = m.layers[li];
    layers[li].k_cache = Ld.k_cache; layers[li].v_cache = Ld.v_cache;
    layers[li].q_gamma = Ld.q_gamma; layers[li].k_gamma = Ld.k_gamma;
    layers[li].cos_t = Ld.cos_t; layers[li].sin_t = Ld.sin_t; layers[li].window = Ld.window;
    const int64_t qkv = (int64_t)(m.nh + 2 * m.nkv) * m.d, hd = (int64_t)m.nh * m.d;
    CG_TRY(gemm_phase(Ld.w_qkv, qkv, m.H, qkv, 0, mx_xn, EP_SCALE_F32, (void*)m.qkv, qkv, nullptr, parts, slot, 0, li));
    RPhase at{};
    at.kind = PH_ATTN; at.layer = li;
    phases.push_back(at);
    CG_TRY(gemm_phase(Ld.w_o, m.H, hd, m.H, 0, mx_att, EP_RESIDUAL, nullptr, m.H, Ld.gain_ffn, 0, 0, slot ^ 1, li));
    CG_TRY(gemm_phase(Ld.w_gu, 2 * (int64_t)m.F, m.H, m.F, 1, mx_xn, EP_ACTMUL, (void*)m.hact, m.F, nullptr, parts_res, slot ^ 1, 0, li));
    const float* next_gain = li + 1 < L ? m.layers[li + 1].gain_in : m.gain_final;
    CG_TRY(gemm_phase(Ld.w_down, m.H, m.F, m.H, 0, mx_h, EP_RESIDUAL, nullptr, m.H, next_gain, 0, 0, slot, li));
    parts = parts_res;
  }
  CG_TRY(gemm_phase(m.head, m.Vp, m.H, m.Vp, 0, mx_xn, EP_HEAD, (void*)m.logits, m.Vp, nullptr, parts, slot, 0, L));
  pl->algorithmic_bytes = bytes;

  // ---- device tables ----
  const size_t ph_bytes = (phases.size() * sizeof(RPhase) + 127) / 128 * 128;
  const size_t ly_bytes = (layers.size() * sizeof(RLayer) + 127) / 128 * 128;
  const size_t mp_bytes = maps.size() * sizeof(CUtensorMap);
  constexpr int TRACE_CAP = 512;
  const size_t total = ph_bytes + ly_bytes + mp_bytes + 128 + (size_t)TRACE_CAP * 16;
  size_t got = 0;
  pl->dev_blob = c->core->alloc(total + 128, &got);
  if (!pl->dev_blob) return fail(c, CG_ERR_OOM, "resident decode: out of device memory");
  pl->algorithmic_bytes = bytes;
  char* basep = (char*)(((uintptr_t)pl->dev_blob + 127) / 128 * 128);
  std::vector<char> host(total, 0);
  memcpy(host.data(), maps.data(), mp_bytes);
  memcpy(host.data() + mp_bytes, phases.data(), phases.size() * sizeof(RPhase));
  memcpy(host.data() + mp_bytes + ph_bytes, layers.data(), layers.size() * sizeof(RLayer));
  CG_CUDA(c, cudaMemcpyAsync(basep, host.data(), total, cudaMemcpyHostToDevice, c->core->stream));
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));  // `host` goes out of scope
  pl->blob_bytes = got;

  RArgs& a = pl->args;
  a.maps = (const CUtensorMap*)basep;
  a.phases = (const RPhase*)(basep + mp_bytes);
  a.layers = (const RLayer*)(basep + mp_bytes + ph_bytes);
  a.bar = (unsigned*)(basep + mp_bytes + ph_bytes + ly_bytes);
  a.trace = nullptr;
  a.trace_cap = TRACE_CAP;
  a.trace_cta = 0;
  a.prefetch_ahead = getenv("CG_RES_PREFETCH") ? atoi(getenv("CG_RES_PREFETCH")) : 0;
  pl->trace_area = (unsigned long long*)(basep + mp_bytes + ph_bytes + ly_bytes + 128);
  a.n_phases = (int)phases.size();
  a.n_steps = 0;
  a.n_clusters = NC;
  a.stages = stages;
  a.gen_bytes = (int)gen;
  // context slices per (row, kv head): enough groups for all pairs in as few rounds as possible
  {
    const int64_t pairs = M * m.nkv;
    int best_g = R_CS;
    double best_cost = 1e30;
    for (int g = 1; g <= R_CS; g *= 2) {
      const int64_t groups = (int64_t)NC * (R_CS / g);
      const int64_t rounds = (pairs + groups - 1) / groups;
      const double cost = (double)rounds * (2.0 + (double)m.Tmax / g / 256.0);
      if (cost < best_cost) { best_cost = cost; best_g = g; }
    }
    a.attn_group = c->opt_res_group ? c->opt_res_group : best_g;
  }
  a.M = (int)M; a.H = (int)m.H; a.nh = m.nh; a.nkv = m.nkv; a.d = m.d; a.qkv_ld = (m.nh + 2 * m.nkv) * m.d;
  a.Tmax = (int)m.Tmax; a.vocab = (int)m.vocab; a.act = m.act; a.plus_one = m.plus_one; a.embed_storage = m.embed_storage;
  a.eps = m.eps; a.attn_scale = 1.0f / sqrtf((float)m.d); a.attn_softcap = m.attn_softcap; a.final_softcap = m.final_softcap;
  a.embed_scale = m.embed_scale;
  a.x = m.x; a.xn = m.xn; a.ss = m.ss; a.ss_stride = m.ss_parts_cap / 2 * 32; a.qkv = m.qkv; a.att = m.att;
  a.embed = m.embed; a.gain0 = m.layers[0].gain_in;
  a.cur = m.cur; a.history = m.history; a.hist_ld = m.hist_ld; a.count_dev = m.count_dev; a.pos_dev = m.pos_dev;
  a.best = m.best; a.err = c->core->dev_err;
  *out = pl.release();
  return CG_OK;
}

int decode_resident_run(cg_ctx* c, ResidentPlan* pl, int n_steps) {
  if (n_steps <= 0) return CG_OK;
  pl->args.n_steps = n_steps;
  CG_CUDA(c, cudaMemsetAsync(pl->args.bar, 0, 4, c->core->stream));
  if (pl->tn == 16 && pl->d == 64) return launch<16, 64>(c, *pl);
  if (pl->tn == 16) return launch<16, 128>(c, *pl);
  if (pl->d == 64) return launch<32, 64>(c, *pl);
  return launch<32, 128>(c, *pl);
}

void decode_resident_free(ResidentPlan* pl) {
  if (!pl) return;
  if (pl->dev_blob) pl->core->recycle(pl->dev_blob, pl->blob_bytes);
  delete pl;
}

int decode_resident_trace(cg_ctx* c, ResidentPlan* pl, int cta, uint64_t* out, int n) {
  if (cta < 0) { pl->args.trace = nullptr; return CG_OK; }
  if (!out) {  // arm: the next run records
    pl->args.trace = pl->trace_area;
    pl->args.trace_cta = cta;
    CG_CUDA(c, cudaMemsetAsync(pl->trace_area, 0, (size_t)pl->args.trace_cap * 16, c->core->stream));
    return CG_OK;
  }
  if (n > pl->args.trace_cap * 2) n = pl->args.trace_cap * 2;
  CG_CUDA(c, cudaMemcpyAsync(out, pl->trace_area, (size_t)n * 8, cudaMemcpyDeviceToHost, c->core->stream));
  CG_CUDA(c, cudaStreamSynchronize(c->core->stream));
  return CG_OK;
}

int64_t decode_resident_bytes_per_step(const ResidentPlan* pl) { return pl ? pl->algorithmic_bytes : 0; }
int decode_resident_grid(const ResidentPlan* pl) { return pl ? pl->grid : 0; }

}  // namespace cg
