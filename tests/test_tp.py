"""Tensor parallelism.  CPU part (gloo, world size 2): shards of the seeded model tile the full model exactly and the
id rendezvous delivers rank 0's bytes.  GPU part (needs two GPUs): a 2-rank run gives the single-GPU logits."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import helpers
from tests.tp_worker import SHAPE

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gloo_worker(rank, world, port, tmp):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from lazyweights_b200 import modelgen
    W = modelgen.write_model(os.path.join(tmp, "s%d" % rank), SHAPE, "Q4_K", "Q6_K", seed=9, tp=(rank, world),
                             return_weights=True)
    # the rendezvous used for the NCCL id: rank 0's 128 bytes must arrive everywhere
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf.copy_(torch.arange(128, dtype=torch.uint8))
    dist.broadcast(buf, src=0)
    assert buf.tolist() == list(range(128))
    np.savez(os.path.join(tmp, "w%d.npz" % rank), **{k: v[1] for k, v in W.items() if not k.startswith("__")})
    dist.barrier()
    dist.destroy_process_group()


def test_shards_tile_the_full_model(tmp_path):
    import torch.multiprocessing as mp
    helpers.build_library()
    mp.spawn(_gloo_worker, args=(2, 29731, str(tmp_path)), nprocs=2, join=True)
    from lazyweights_b200 import modelgen
    full = modelgen.write_model(str(tmp_path / "full"), SHAPE, "Q4_K", "Q6_K", seed=9, return_weights=True)
    s = [np.load(tmp_path / ("w%d.npz" % r)) for r in range(2)]
    H, Hk, Dh = SHAPE["n_heads"], SHAPE["n_kv_heads"], SHAPE["head_dim"]
    for l in range(SHAPE["n_layers"]):
        q = full["l%d.qkv" % l][1]
        parts = [s[r]["l%d.qkv" % l] for r in range(2)]
        hq, hk = H // 2 * Dh, Hk // 2 * Dh
        rebuilt = np.concatenate([parts[0][:hq], parts[1][:hq], parts[0][hq:hq + hk], parts[1][hq:hq + hk],
                                  parts[0][hq + hk:], parts[1][hq + hk:]])
        assert np.array_equal(rebuilt, q)
        for name, axis in (("o", 1), ("gate", 0), ("up", 0), ("down", 1)):
            key = "l%d.%s" % (l, name)
            assert np.array_equal(np.concatenate([s[0][key], s[1][key]], axis), full[key][1])
    assert np.array_equal(np.concatenate([s[0]["lm_head"], s[1]["lm_head"]]), full["lm_head"][1])


@pytest.mark.gpu
@pytest.mark.parametrize("peer", ["1", "0"])
def test_two_rank_forward_matches_one_gpu(tmp_path, peer):
    """peer = 1: all-reduces over peer memory fused with the norm; 0: NCCL all-reduces."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    helpers.build_library()
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29741" if peer == "1" else "29743", WORLD_SIZE="2",
               NCCL_NVLS_ENABLE="0", LW_TP_PEER=peer)
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "tp_worker.py"), str(tmp_path)],
                              env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
             for r in range(2)]
    outs = [p.communicate(timeout=600)[0].decode() for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    modelgen.write_model(str(tmp_path / "full"), SHAPE, "Q4_K", "Q6_K", seed=9)
    ids = np.random.default_rng(2).integers(0, SHAPE["vocab"], 10).astype(np.int32)
    with lw.Bundle(str(tmp_path / "full"), max_ctx=64, max_batch=8) as b:
        ref = b.forward(ids, all_logits=True)
        ref_step = b.forward(ids[:1])
    for r in range(2):
        assert helpers.rel_err(np.load(tmp_path / ("logits%d.npy" % r)), ref) <= 1e-3
        assert helpers.rel_err(np.load(tmp_path / ("step%d.npy" % r)), ref_step) <= 1e-3


def test_uneven_split_over_eight_ranks(tmp_path):
    """A paired 4-bit FFN of 7 tile columns and a vocabulary of 13 tile rows over 4 ranks: 2, 2, 2, 1 tile columns and
    4, 3, 3, 3 tile rows; the shards must tile the full model and every shard must validate (host only)."""
    helpers.build_library()
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen
    assert [modelgen.tile_split(14336, 512, 8, r) for r in (0, 3, 4, 7)] == [(0, 2048), (6144, 8192), (8192, 9728), (12800, 14336)]
    assert [modelgen.tile_split(32000, 64, 8, r)[1] - modelgen.tile_split(32000, 64, 8, r)[0] for r in range(8)] == [4032] * 4 + [3968] * 4
    shape = dict(SHAPE, inter=7 * 512, vocab=13 * 64, n_heads=16, n_kv_heads=4, n_layers=1)
    full = modelgen.write_model(str(tmp_path / "full"), shape, "Q4_K", "Q4_K", seed=2, return_weights=True)
    parts = []
    for r in range(4):
        path = str(tmp_path / ("s%d" % r))
        parts.append(modelgen.write_model(path, shape, "Q4_K", "Q4_K", seed=2, tp=(r, 4), return_weights=True))
        assert lw.lib().lw_validate_bundle(path.encode()) == 0, lw._native.last_error()
        cfg, _ = lw.bundle.read_manifest(path)
        assert int(cfg["vocab_full"]) == shape["vocab"] and int(cfg["inter"]) == parts[-1]["l0.gate"][1].shape[0]
    assert [p["l0.gate"][1].shape[0] // 512 for p in parts] == [2, 2, 2, 1]
    assert [p["lm_head"][1].shape[0] // 64 for p in parts] == [4, 3, 3, 3]
    for name, axis in (("gate", 0), ("up", 0), ("down", 1)):
        key = "l0." + name
        assert np.array_equal(np.concatenate([p[key][1] for p in parts], axis), full[key][1])
        assert np.array_equal(np.concatenate([p[key][2] for p in parts], axis), full[key][2])   # side bytes too
    assert np.array_equal(np.concatenate([p["lm_head"][1] for p in parts]), full["lm_head"][1])


HEARTBEAT_WORKER = r"""
import sys, time
sys.path.insert(0, %r)
import torch.distributed as dist
from lazyweights_b200.tp import Heartbeat, PeerLost
rank, port, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
store = dist.TCPStore("127.0.0.1", port, 2, rank == 0, timeout=__import__("datetime").timedelta(seconds=20))
hb = Heartbeat(store, rank, 2, timeout_s=1.0)
log = []
for step in range(4):
    if rank == 1 and step == 2:
        log.append("left before step 2")          # leaves between steps: nothing of its own is in flight
        break
    t0 = time.monotonic()
    try:
        hb.before_step(step)
        log.append("step %%d ok" %% step)
    except PeerLost as e:
        log.append("step %%d lost %%s after %%.1f s" %% (e.step, e.missing, time.monotonic() - t0))
        break
open(out, "w").write("\n".join(log))
if rank == 0:
    time.sleep(0.3)                                # the store lives in rank 0: let the peer finish its last read
"""


def test_rank_that_leaves_between_steps_is_noticed_on_the_host(tmp_path):
    """Failure detection without a GPU and without a fault: two processes share a TCP store; rank 1 stops after two
    steps; rank 0 learns of it on the host, within the heartbeat's timeout, before it launches step 2."""
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = HEARTBEAT_WORKER % (ROOT,)
    procs = [subprocess.Popen([sys.executable, "-c", script, str(r), str(port), str(tmp_path / ("r%d.log" % r))])
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=120) == 0
    log0 = (tmp_path / "r0.log").read_text().splitlines()
    log1 = (tmp_path / "r1.log").read_text().splitlines()
    assert log1 == ["step 0 ok", "step 1 ok", "left before step 2"]
    assert log0[:2] == ["step 0 ok", "step 1 ok"]
    assert log0[2].startswith("step 2 lost [1] after 1.")


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_reports(tmp_path):
    """The wait at the end of a tensor-parallel pass is bounded: with the stream held up by a sleeping host function
    (the GPU idle, nothing faults) a 100 ms bound gives up and reports, a 2 s bound sees the stream drain."""
    helpers.build_library()
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen
    from tests.test_runtime import SHAPE
    modelgen.write_model(str(tmp_path / "m"), SHAPE, "Q4_K", "Q4_K", seed=3)
    with lw.Bundle(str(tmp_path / "m"), max_ctx=64, max_batch=8) as b:
        b.tp_set_timeout(2000)
        assert b.debug_stream_stall(300) == 0
        b.tp_set_timeout(100)
        assert b.debug_stream_stall(600) == -4                          # gave up after 100 ms
        from lazyweights_b200 import _native as nat
        assert "did not finish within 100 ms" in nat.last_error()
        b.tp_set_timeout(0)
        ok = b.forward(np.array([1, 2, 3], np.int32))                    # a handle without peers lost nothing
        assert np.isfinite(ok).all()
