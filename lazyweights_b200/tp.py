"""Tensor-parallel helpers: one process per GPU, torch.distributed for the rendezvous, NCCL inside the library.

Each rank opens its own shard bundle (see modelgen.write_model(tp=(rank, world))).  Rank 0 asks the library for an
NCCL unique id, the id travels to the other ranks through the already-initialised torch.distributed group (gloo or
nccl), and every rank hands it to rt_tp_init.  After that rt_forward all-reduces the partial outputs of the
row-parallel matrices (o, down) and gathers the logits slices.
"""
import numpy as np

from .runtime import Bundle, tp_unique_id


def broadcast_id(rank, group=None, device=None):
    """The 128-byte NCCL id of rank 0, delivered to every rank of the torch.distributed group."""
    import torch
    import torch.distributed as dist
    buf = torch.zeros(128, dtype=torch.uint8, device=device or "cpu")
    if rank == 0:
        buf.copy_(torch.frombuffer(bytearray(tp_unique_id()), dtype=torch.uint8))
    dist.broadcast(buf, src=0, group=group)
    return bytes(buf.cpu().numpy().tobytes())


def open_shard(path, rank, world, max_ctx=4096, max_batch=8, group=None, device=None):
    """Opens this rank's shard bundle on the current CUDA device and joins the tensor-parallel communicator."""
    b = Bundle(path, max_ctx=max_ctx, max_batch=max_batch)
    if world > 1:
        b.tp_init(rank, world, broadcast_id(rank, group, device))
    return b
