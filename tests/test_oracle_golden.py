"""The CPU oracle against vectors written by the reference's own Python code (tests/golden)."""
import glob
import os

import numpy as np
import pytest

from oracle import lw_oracle as orc

HISTS = ["geometric", "flat64", "ties", "random256", "sparse", "single", "fib"]
FORMATS = ["Q4_K_128x1024", "Q5_K_128x512", "Q6_K_192x512", "IQ4_XS_64x1536"]
EDGES = ["single", "uniform256", "two", "skewed"]


@pytest.mark.parametrize("name", HISTS)
def test_tables_match_reference(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "tables.npz"))
    hist = g[name + "_hist"]
    assert np.array_equal(orc.huffman_lengths(hist), g[name + "_plain"])
    lim = orc.limited_lengths(hist)
    assert np.array_equal(lim, g[name + "_limited"])
    assert lim.max() <= 11
    assert np.array_equal(orc.canonical_codes(lim), g[name + "_codes"])
    lut = orc.build_lut(lim)
    assert np.array_equal(lut, g[name + "_lut"])
    assert np.array_equal(orc.lengths_from_lut(lut), lim.astype(np.int64))


@pytest.mark.parametrize("name", HISTS)
def test_comparator_equals_table(golden_dir, name):
    """The limit-register form must resolve every window the table resolves, to the same (symbol, length)."""
    g = np.load(os.path.join(golden_dir, "tables.npz"))
    lut = g[name + "_lut"]
    tabs = orc.comparator_tables(lut)
    for w in range(0, 2048, 1 if name != "random256" else 3):
        if lut[w] >> 8 == 0:
            continue                      # only the single-symbol table has unresolved windows
        assert orc.comparator_lookup(tabs, w) == (int(lut[w] & 255), int(lut[w] >> 8))


@pytest.mark.parametrize("name", FORMATS)
def test_block_formats_match_reference(golden_dir, name):
    ty = name.rsplit("_", 1)[0]
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    q, side, blocks = g["q"], g["side"], g["blocks"]
    n, k = q.shape
    q2, side2 = orc.split_blocks(ty, blocks)
    assert np.array_equal(q2.reshape(n, k), q)
    assert np.array_equal(side2.reshape(n, -1), side)
    assert np.array_equal(orc.join_blocks(ty, q.reshape(-1, 256), side.reshape(n * k // 256, -1)), blocks)
    w = orc.dequant(ty, q, side)
    assert w.dtype == np.float32 and np.array_equal(w, g["w"])           # bit-exact, gguf-py == reference
    sym = orc.symbols_of(ty, q)
    assert np.array_equal(sym, g["sym"])
    assert np.array_equal(orc.codes_of(ty, sym), q)
    blob, nbits, hist = orc.encode_huf8(sym)
    assert nbits == int(g["nbits"]) and np.array_equal(hist, g["hist"])
    assert blob == g["blob"].tobytes()                                     # the encoder is byte-exact
    assert np.array_equal(orc.decode_huf8(g["blob"].tobytes(), *sym.shape), g["decoded"])
    y = orc.gemv_f64(w, g["x"].astype(np.float32))
    assert np.allclose(y, g["y"], rtol=1e-12, atol=0)


@pytest.mark.parametrize("name", EDGES)
def test_edge_blobs_match_reference(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "edge_%s.npz" % name))
    sym = g["sym"]
    blob, nbits, hist = orc.encode_huf8(sym)
    assert nbits == int(g["nbits"])
    assert blob == g["blob"].tobytes()
    assert np.array_equal(orc.decode_huf8(blob, *sym.shape), sym)
    lut = np.frombuffer(blob, np.uint16, 2048)
    if name == "single":
        assert nbits == sym.size and (lut >> 8).max() == 1 and (lut[1::2] == 0).all()
    if name == "skewed":
        assert (lut >> 8).max() == 11


def test_stream_order_roundtrip():
    rng = np.random.default_rng(3)
    sym = rng.integers(0, 256, (192, 768)).astype(np.uint8)
    flat = orc.to_stream_order(sym)
    assert np.array_equal(orc.from_stream_order(flat, 192, 768), sym)
    # lane 5 of tile (row 1, column 2): tile rows 5 and 37
    t = 1 * 3 + 2
    lane = flat.reshape(-1, 32, 2, 256)[t, 5]
    assert np.array_equal(lane[0], sym[64 + 5, 512:768]) and np.array_equal(lane[1], sym[64 + 37, 512:768])


def test_bundle_files(tmp_path):
    rng = np.random.default_rng(5)
    w = orc.BundleWriter(str(tmp_path / "b"))
    w.cfg("hidden", 512)
    q = orc.synth_codes("Q6_K", 64, 512, rng)
    side = orc.synth_side("Q6_K", 64, 512, rng)
    w.add_matrix("l0.up", "Q6_K", q, side)
    w.close()
    cfg, ts = orc.read_manifest(str(tmp_path / "b"))
    assert cfg == {"hidden": "512"} and [t["name"] for t in ts] == ["l0.up", "l0.up.kqs"]
    assert ts[0]["enc"] == "huf8" and ts[1]["enc"] == "kq_Q6_K" and ts[1]["K"] == 2 * 18
    assert all(t["offset"] % 256 == 0 for t in ts)
    raw = open(tmp_path / "b" / "weights.bin", "rb").read()
    blob = raw[ts[0]["offset"]:ts[0]["offset"] + ts[0]["nbytes"]]
    assert np.array_equal(orc.decode_huf8(blob, 64, 512), q)
