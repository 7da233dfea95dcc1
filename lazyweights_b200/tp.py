"""Tensor-parallel helpers: one process per GPU, torch.distributed for the rendezvous, NCCL inside the library.

Each rank opens its own shard bundle (see modelgen.write_model(tp=(rank, world))).  Rank 0 asks the library for an
NCCL unique id, the id travels to the other ranks through the already-initialised torch.distributed group (gloo or
nccl), and every rank hands it to rt_tp_init.  After that rt_forward all-reduces the partial outputs of the
row-parallel matrices (o, down) and gathers the logits slices.
"""
import time

import numpy as np

from .runtime import Bundle, tp_unique_id


class PeerLost(RuntimeError):
    """A rank did not reach the step the others are about to launch."""

    def __init__(self, step, missing):
        super().__init__("ranks %s did not reach step %d" % (missing, step))
        self.step, self.missing = step, missing


class Heartbeat:
    """Host-side liveness check between steps.  Every rank announces the step it is about to launch in a key-value
    store (a torch.distributed TCPStore / FileStore, or anything with set / get of byte strings) and looks at its
    peers' announcements before it launches: a rank that left - between steps, with nothing of its own in flight - is
    noticed here, on the host, within `timeout_s`, instead of inside a collective that would never complete.  (The
    library's own bound on a pass, rt_tp_set_timeout, covers a rank lost in the middle of a step.)"""

    def __init__(self, store, rank, world, timeout_s=5.0, poll_s=0.005):
        self.store, self.rank, self.world, self.timeout_s, self.poll_s = store, rank, world, timeout_s, poll_s

    def _key(self, rank):
        return "lwb200/step/%d" % rank

    def announce(self, step):
        self.store.set(self._key(self.rank), str(int(step)))

    def reached(self, rank):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return -1                            # a TCPStore's get would block for the key
            return int(bytes(self.store.get(self._key(rank))).decode())
        except Exception:                            # no announcement yet
            return -1

    def before_step(self, step):
        """Announces `step` and waits until every rank has announced it; raises PeerLost after timeout_s."""
        self.announce(step)
        deadline = time.monotonic() + self.timeout_s
        while True:
            missing = [r for r in range(self.world) if r != self.rank and self.reached(r) < step]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise PeerLost(step, missing)
            time.sleep(self.poll_s)


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
