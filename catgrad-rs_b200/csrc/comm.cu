// comm.cu — tensor-parallel communicator: NCCL over NVLink/NVSwitch, one process per GPU.
// The unique id is created on rank 0 and carried to the other ranks by the caller (the
// Python side broadcasts it through torch.distributed); collectives run on the context's
// stream so they order with the kernels around them and can be captured in CUDA graphs.
#include <cstring>

#include "nccl_dl.h"
#include "runtime.h"

using namespace cg;

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
  return CG_OK;
}

int32_t cg_comm_destroy(cg_ctx* c) {
  if (!c) return CG_ERR_INVALID;
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
  ncclResult_t r = nccl().AllReduce(t->data(), t->data(), (size_t)t->numel(), dt, ncclSum, (ncclComm_t)c->comm, c->core->stream);
  if (r != ncclSuccess) return fail(c, CG_ERR_COMM, std::string("ncclAllReduce: ") + nccl().GetErrorString(r));
  return CG_OK;
}

}  // extern "C"
