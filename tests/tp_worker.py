"""Worker of the tensor-parallel test: one process per GPU.  argv: out_dir.  Env: RANK, WORLD_SIZE, MASTER_*."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHAPE = dict(n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=128, inter=2048, vocab=1024, eps=1e-5, theta=1e4)


def main():
    import torch
    import torch.distributed as dist
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen, tp
    out = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")
    path = os.path.join(out, "shard%d" % rank)
    modelgen.write_model(path, SHAPE, "Q4_K", "Q6_K", seed=9, tp=(rank, world))
    ids = np.random.default_rng(2).integers(0, SHAPE["vocab"], 10).astype(np.int32)
    b = tp.open_shard(path, rank, world, max_ctx=64, max_batch=8)
    logits = b.forward(ids, all_logits=True)
    step = b.forward(ids[:1])                      # one more single-token pass (m = 1 path through the collectives)
    assert b.kernel_error() == 0 and b.tp_error() == 0
    np.save(os.path.join(out, "logits%d.npy" % rank), logits)
    np.save(os.path.join(out, "step%d.npy" % rank), step)
    dist.barrier()
    b.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
