"""Tensor parallelism of the decoder over the GPUs of one node: one process per GPU.

The model shards where it does naturally (attention heads and FFN columns are independent
until the output projections, the vocabulary until the arg-max):

* q/k/v projections: rows of the rank's heads            (column parallel)
* o projection:      columns of the rank's heads         (row parallel  -> all-reduce)
* gate/up:           rows of the rank's FFN slice        (column parallel)
* down:              columns of the rank's FFN slice     (row parallel  -> all-reduce)
* LM head:           rows of the rank's vocabulary slice (all-gather of logits, then arg-max)
* experts:           whole experts per rank; every rank routes all tokens, runs the experts it
                     owns, and the partial sums meet in the same all-reduce as a row-parallel GEMM

`shard_plan` is the index arithmetic (the native decoder applies the same ranges when it
keeps its shard of the full tensors it is handed); `init_comm` carries the NCCL unique id
from rank 0 to the others through torch.distributed.
"""
from __future__ import annotations

import ctypes as C


def shard_plan(cfg, rank: int, world: int) -> dict:
    """Row/column ranges (start, stop) of every sharded parameter for `rank` of `world`."""
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.get_head_dim()
    F, V = cfg.intermediate_size, cfg.vocab_size
    E = getattr(cfg, "num_local_experts", 0)
    # fewer kv heads than ranks: every kv head is replicated on world / nkv consecutive ranks
    kv_ok = nkv % world == 0 or (nkv < world and world % nkv == 0)
    if nh % world or not kv_ok or F % world or V % world or (E > 1 and E % world):
        raise ValueError("heads, kv heads, ffn, vocab and experts must divide by the tensor-parallel degree")
    q = (rank * (nh // world) * d, (rank + 1) * (nh // world) * d)
    if nkv >= world:
        kv = (rank * (nkv // world) * d, (rank + 1) * (nkv // world) * d)
    else:
        head = rank * nkv // world  # the kv head this rank's query heads belong to
        kv = (head * d, (head + 1) * d)
    f = (rank * (F // world), (rank + 1) * (F // world))
    v = (rank * (V // world), (rank + 1) * (V // world))
    plan = {"q_rows": q, "kv_rows": kv, "o_cols": q, "ffn_rows": f, "down_cols": f, "vocab_rows": v}
    if E > 1:
        plan["experts"] = (rank * (E // world), (rank + 1) * (E // world))  # whole experts per rank
    return plan


def init_comm(backend, rank: int, world: int) -> None:
    """Create the library's NCCL communicator on `backend` (collective over all ranks).
    torch.distributed must already be initialised; it only moves the 128-byte id."""
    import torch
    import torch.distributed as dist

    L = backend._lib
    L.cg_comm_id_size.restype = C.c_int32
    L.cg_comm_make_id.argtypes = [C.c_void_p]
    L.cg_comm_init.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]
    n = L.cg_comm_id_size()
    raw = (C.c_uint8 * n)()
    if rank == 0:
        if L.cg_comm_make_id(raw) != 0:
            raise RuntimeError("cg_comm_make_id failed")
    buf = torch.tensor(list(raw), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        buf = buf.cuda()
    dist.broadcast(buf, 0)
    raw = (C.c_uint8 * n)(*buf.cpu().tolist())
    backend._check(L.cg_comm_init(backend._ctx, raw, int(rank), int(world)))
