"""Writes the golden fixtures of this directory by running the REFERENCE project's own Python code.

Run it where a checkout of the reference is available (it is imported in place, nothing is copied):

    python tests/golden/make_golden.py <path-to-reference-checkout>

It needs numpy and the `gguf` package.  Outputs (all small, seeded, deterministic):
  tables.npz                 code-length and table known answers (plain, halved-count, degenerate histograms)
  <TYPE>_<N>x<K>.npz         per block format: codes, side bytes, GGUF block bytes, symbols, the blob of the
                             reference encoder, the reference decoder's output, float32 weights from the
                             reference's kernel-arithmetic restatement and from gguf-py (identical)
  edge_*.npz                 single-symbol matrix, all-256-symbols-uniform matrix (every code 8 bits),
                             a skewed matrix whose longest code reaches the 11-bit limit
The tests compare the oracle and the CUDA path against these files; they never need the reference itself.
"""
import os
import sys

import numpy as np


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LW_REFERENCE", "")
    if not ref:
        sys.exit("usage: make_golden.py <reference checkout>   (or set LW_REFERENCE)")
    ref = os.path.abspath(ref)
    out = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ref, "scripts"))
    import gguf
    from lazyweights import bundle, huffman, lanecodecs
    import kq_code
    import a2_kq_bundle as kqb

    T = gguf.GGMLQuantizationType
    types = {"Q4_K": T.Q4_K, "Q5_K": T.Q5_K, "Q6_K": T.Q6_K, "IQ4_XS": T.IQ4_XS}
    sys.path.insert(0, os.path.join(out, "..", ".."))
    from oracle import lw_oracle as orc          # only its seeded input generators are used here

    # ---- tables ------------------------------------------------------------------------------------
    rng = np.random.default_rng(11)
    hists = {
        "geometric": (1 << np.arange(24))[::-1].astype(np.int64),                    # forces count halving
        "flat64": np.full(64, 1000, np.int64),
        "ties": np.array([5, 5, 5, 5, 3, 3, 2, 2, 1, 1, 1, 1, 1], np.int64),
        "random256": rng.integers(1, 100000, 256).astype(np.int64),
        "sparse": np.where(rng.random(256) < 0.2, rng.integers(1, 1 << 20, 256), 0).astype(np.int64),
        "single": np.eye(1, 256, 77, dtype=np.int64)[0] * 12345,
        "fib": np.array([1, 1, 2, 3, 5, 8, 13, 21, 34, 55, 89, 144, 233, 377, 610, 987, 1597, 2584], np.int64),
    }
    tab = {}
    for name, h in hists.items():
        h256 = np.zeros(256, np.int64)
        h256[:h.size] = h
        tab[name + "_hist"] = h256
        tab[name + "_plain"] = huffman.code_lengths(h256)
        lim = lanecodecs.limited_lengths(h256, 11)
        tab[name + "_limited"] = lim
        tab[name + "_codes"] = lanecodecs.canonical_codes(lim)
        tab[name + "_lut"] = bundle.build_lut(lim)
    np.savez_compressed(os.path.join(out, "tables.npz"), **tab)

    # ---- block formats ---------------------------------------------------------------------------
    shapes = {"Q4_K": (128, 1024), "Q5_K": (128, 512), "Q6_K": (192, 512), "IQ4_XS": (64, 1536)}
    for seed, (name, ty) in enumerate(types.items()):
        n, k = shapes[name]
        rng = np.random.default_rng(100 + seed)
        q = orc.synth_codes(name, n, k, rng)
        side = orc.synth_side(name, n, k, rng)
        blocks = kq_code.join(ty, q.reshape(-1, 256), side.reshape(n * k // 256, -1))
        q2, side2, _ = kq_code.split(ty, blocks)
        assert np.array_equal(q2.reshape(n, k), q) and np.array_equal(side2.reshape(n, -1), side)
        w_kernel = kqb.dequant(ty, q, side)
        w_gguf = gguf.quants.dequantize(blocks.reshape(n, -1), ty).reshape(n, k)
        assert np.array_equal(w_kernel, w_gguf), name
        sym = q if kqb.BITS[ty] == 8 else np.ascontiguousarray(q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
        blob, nbits, hist = bundle.encode_huf8(sym)
        dec = bundle.decode_huf8(blob, *sym.shape)
        assert np.array_equal(dec, sym)
        x = rng.standard_normal((8, k)).astype(np.float16)
        np.savez_compressed(os.path.join(out, "%s_%dx%d.npz" % (name, n, k)), q=q, side=side, blocks=blocks,
                            sym=sym, blob=np.frombuffer(blob, np.uint8), nbits=np.int64(nbits), hist=hist,
                            decoded=dec, w=w_gguf, x=x,
                            y=x.astype(np.float64) @ w_gguf.astype(np.float64).T)

    # ---- edge cases ------------------------------------------------------------------------------
    rng = np.random.default_rng(7)
    edge = {
        "single": np.full((64, 256), 200, np.uint8),
        "uniform256": rng.integers(0, 256, (64, 512)).astype(np.uint8),
        "two": rng.integers(0, 2, (64, 256)).astype(np.uint8) * 255,
    }
    p = 0.5 ** np.arange(1, 41)
    p /= p.sum()
    edge["skewed"] = rng.choice(40, (128, 256), p=p).astype(np.uint8)               # longest code = 11 bits
    for name, sym in edge.items():
        blob, nbits, hist = bundle.encode_huf8(sym)
        dec = bundle.decode_huf8(blob, *sym.shape)
        assert np.array_equal(dec, sym), name
        np.savez_compressed(os.path.join(out, "edge_%s.npz" % name), sym=sym, blob=np.frombuffer(blob, np.uint8),
                            nbits=np.int64(nbits), hist=hist, decoded=dec)
    print("golden fixtures written to", out)


if __name__ == "__main__":
    main()
