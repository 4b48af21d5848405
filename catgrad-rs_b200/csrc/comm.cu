// comm.cu — tensor-parallel communicator: NCCL over NVLink/NVSwitch, one process per GPU.
// The unique id is created on rank 0 and carried to the other ranks by the caller (the
// Python side broadcasts it through torch.distributed); collectives run on the context's
// stream so they order with the kernels around them and can be captured in CUDA graphs.
#include <cstdio>
#include <cstring>
#include <vector>

#include "nccl_dl.h"
#include "runtime.h"

using namespace cg;

namespace {

constexpr int64_t XCHG_MAX_ELEMS = 32 * 8192;   // 32 tokens of hidden size 8192
constexpr size_t XCHG_FLAG_BYTES = 4096;        // flags, epoch, ticket

size_t xchg_bytes(int world) { return XCHG_FLAG_BYTES + (size_t)2 * world * XCHG_MAX_ELEMS * 4; }

void xchg_close(cg_ctx* c) {
  PeerXchg& x = c->xchg;
  for (int r = 0; r < MAX_PEERS; ++r)
    if (x.opened[r]) { cudaIpcCloseMemHandle(x.opened[r]); x.opened[r] = nullptr; }
  if (x.local_base) { cudaFree(x.local_base); x.local_base = nullptr; }
  x.ok = false;
}

// Allocates this rank's exchange area, trades inter-process handles through the NCCL
// communicator and maps every peer's area.  On failure the communicator stays usable and the
// callers keep to NCCL collectives; `why` says what happened.
void xchg_setup(cg_ctx* c, int rank, int world) {
  PeerXchg& x = c->xchg;
  x.ok = false;
  x.world = world;
  x.rank = rank;
  x.max_elems = XCHG_MAX_ELEMS;
  if (world < 2 || world > MAX_PEERS) { x.why = "world size outside [2, 8]"; return; }
  // Every rank walks through the same two collectives whatever fails locally, so a failure on
  // one rank can neither hang the others nor leave them believing the exchange works.
  const size_t bytes = xchg_bytes(world);
  cudaStream_t s = c->core->stream;
  bool good = true;
  auto bad = [&](const char* what, cudaError_t e) {
    if (good) x.why = std::string(what) + ": " + cudaGetErrorString(e);
    good = false;
    cudaGetLastError();
  };
  cudaError_t e = cudaMalloc(&x.local_base, bytes);
  if (e != cudaSuccess) { x.local_base = nullptr; bad("cudaMalloc", e); }
  if (good && (e = cudaMemset(x.local_base, 0, bytes)) != cudaSuccess) bad("cudaMemset", e);
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  if (good && (e = cudaIpcGetMemHandle(&mine, x.local_base)) != cudaSuccess) bad("cudaIpcGetMemHandle", e);
  // 1: all-gather the handles (64 bytes each) with the communicator that was just created
  void* dev = nullptr;
  std::vector<cudaIpcMemHandle_t> all((size_t)world);
  bool coll = cudaMalloc(&dev, sizeof(mine) * (size_t)(world + 1)) == cudaSuccess;
  coll = coll && cudaMemcpyAsync(dev, &mine, sizeof(mine), cudaMemcpyHostToDevice, s) == cudaSuccess;
  coll = coll && nccl().AllGather(dev, (char*)dev + sizeof(mine), sizeof(mine), ncclChar, (ncclComm_t)c->comm, s) == ncclSuccess;
  coll = coll && cudaMemcpyAsync(all.data(), (char*)dev + sizeof(mine), sizeof(mine) * (size_t)world, cudaMemcpyDeviceToHost, s) == cudaSuccess;
  coll = coll && cudaStreamSynchronize(s) == cudaSuccess;
  if (!coll) { x.why = "exchange of the memory handles failed"; good = false; }
  for (int r = 0; r < world && good; ++r) {
    void* base = x.local_base;
    if (r != rank) {
      e = cudaIpcOpenMemHandle(&base, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) { bad("cudaIpcOpenMemHandle", e); break; }
      x.opened[r] = base;
    }
    x.flags[r] = (uint32_t*)base;
    x.data[r] = (float*)((char*)base + XCHG_FLAG_BYTES);
  }
  if (good) {
    x.epoch = (uint32_t*)((char*)x.local_base + 2048);
    x.ticket = (unsigned*)((char*)x.local_base + 2048 + 128);
  }
  // 2: count the ranks that mapped everything; also the barrier before the first push
  float votes = 0.f;
  if (coll && dev) {
    const float one = good ? 1.f : 0.f;
    coll = cudaMemcpyAsync(dev, &one, 4, cudaMemcpyHostToDevice, s) == cudaSuccess &&
           nccl().AllReduce(dev, dev, 1, ncclFloat32, ncclSum, (ncclComm_t)c->comm, s) == ncclSuccess &&
           cudaMemcpyAsync(&votes, dev, 4, cudaMemcpyDeviceToHost, s) == cudaSuccess && cudaStreamSynchronize(s) == cudaSuccess;
  }
  if (dev) cudaFree(dev);
  if (!coll || votes != (float)world) {
    if (good) x.why = "another rank could not map the exchange area";
    xchg_close(c);
    return;
  }
  x.ok = true;
}

}  // namespace

extern "C" {

int32_t cg_comm_id_size(void) { return (int32_t)sizeof(ncclUniqueId); }

int32_t cg_comm_make_id(void* id_bytes) {
  if (!id_bytes) return CG_ERR_INVALID;
  if (!nccl().ok) return CG_ERR_COMM;
  ncclUniqueId id;
  if (nccl().GetUniqueId(&id) != ncclSuccess) return CG_ERR_COMM;
  memcpy(id_bytes, &id, sizeof(id));
  return CG_OK;
}

int32_t cg_comm_init(cg_ctx* c, const void* id_bytes, int32_t rank, int32_t world) {
  if (!c || !id_bytes || world < 1 || rank < 0 || rank >= world) return fail(c, CG_ERR_INVALID, "bad communicator arguments");
  if (c->comm) return fail(c, CG_ERR_INVALID, "communicator already initialised");
  if (!nccl().ok) return fail(c, CG_ERR_COMM, "libnccl.so.2 could not be loaded");
  CG_CUDA(c, cudaSetDevice(c->core->device));
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  ncclComm_t comm;
  ncclResult_t r = nccl().CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclCommInitRank: ") + nccl().GetErrorString(r));
  c->comm = comm;
  c->comm_rank = rank;
  c->comm_world = world;
  if (world > 1) xchg_setup(c, rank, world);
  return CG_OK;
}

int32_t cg_comm_peer_exchange(cg_ctx* c, char* why, int64_t why_cap) {
  if (!c) return 0;
  if (why && why_cap > 0) snprintf(why, (size_t)why_cap, "%s", c->xchg.ok ? "" : c->xchg.why.c_str());
  return c->xchg.ok ? 1 : 0;
}

int32_t cg_comm_destroy(cg_ctx* c) {
  if (!c) return CG_ERR_INVALID;
  if (c->xchg.local_base) {
    cudaStreamSynchronize(c->core->stream);
    xchg_close(c);
  }
  if (c->comm) {
    nccl().CommDestroy((ncclComm_t)c->comm);
    c->comm = nullptr;
    c->comm_world = 1;
    c->comm_rank = 0;
  }
  return CG_OK;
}

int32_t cg_comm_all_reduce(cg_ctx* c, cg_tensor* t) {
  if (!c || !t) return fail(c, CG_ERR_INVALID, "null argument");
  if (!c->comm) return c->comm_world == 1 ? CG_OK : fail(c, CG_ERR_COMM, "communicator not initialised");
  if (t->tag != CG_F32 || !t->contiguous()) return fail(c, CG_ERR_UNSUPPORTED, "all_reduce wants a contiguous F32-tagged tensor");
  ncclDataType_t dt = t->storage == ST_BF16 ? ncclBfloat16 : ncclFloat32;
  if (t->buf) t->buf->bf16_copy.reset();  // written in place: a cached GEMM operand copy is stale
  ncclResult_t r = nccl().AllReduce(t->data(), t->data(), (size_t)t->numel(), dt, ncclSum, (ncclComm_t)c->comm, c->core->stream);
  if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllReduce: ") + nccl().GetErrorString(r));
  return CG_OK;
}

}  // extern "C"
