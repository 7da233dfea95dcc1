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


def gather_bytes(mine, world, group=None, device=None):
    """Every rank's byte string (all of one length), rank-major, through the torch.distributed group."""
    import torch
    import torch.distributed as dist
    t = torch.frombuffer(bytearray(mine), dtype=torch.uint8).to(device or "cpu")
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t, group=group)
    return b"".join(bytes(p.cpu().numpy().tobytes()) for p in parts)


def open_shard(path, rank, world, max_ctx=4096, max_batch=8, group=None, device=None, peer=None):
    """Opens this rank's shard bundle on the current CUDA device and joins the tensor-parallel communicator.
    peer (default: on unless LW_TP_PEER=0): the all-reduces run over peer memory fused with the following norm
    (rt_tp_peer_export / rt_tp_peer_open) instead of as NCCL calls."""
    import os
    b = Bundle(path, max_ctx=max_ctx, max_batch=max_batch)
    if world > 1:
        b.tp_init(rank, world, broadcast_id(rank, group, device))
        if peer is None:
            peer = os.environ.get("LW_TP_PEER", "1") != "0"
        if peer:
            b.tp_peer_open(gather_bytes(b.tp_peer_export(), world, group, device), world)
    return b
