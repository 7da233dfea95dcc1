"""Random-init decoder bundles in the runtime's bundle format (for tests, benchmarks and dry runs without a GGUF).

Writes what the reference's bundle builder writes for a real model (scripts/a2_kq_bundle.py:152-218): cfg keys,
`embed`, `cos` / `sin` rotary tables computed in float64 (:183-185), `l<i>.ln1/.ln2`, `lnf`, the coded matrices
`l<i>.qkv / .o / .gate / .up / .down`, `lm_head` and their `.kqs` side tensors - with seeded synthetic codes instead of
a quantised checkpoint.  Code distributions per block format: Q4_K Laplace(8, 1.5), IQ4_XS Laplace(7.5, 1.5),
Q5_K N(16, 2.5), Q6_K N(32, 5), clipped to the format's range; fp16 d / dmin ~ U(1e-3, 1e-2); other side bytes uniform.
The embedding is stored as fp16 (`enc f16`, an extension of the format for random-init models).

`reuse_layers=True` writes the matrices of layer 0 once and lets every layer's manifest entry point at the same bytes:
the loader still gives each layer its own device copy, so HBM traffic is that of a full model while the file stays small.
Tensor parallel shards: `tp=(rank, world)` slices heads, FFN width and vocabulary Megatron-style (column-parallel qkv,
gate, up, lm_head; row-parallel o, down) from the same seeded full model, so that shards of different world sizes
describe one model.  FFN width and vocabulary are dealt in whole tiles, as evenly as they go (`tile_split`): a paired
4-bit FFN of width 14336 has 28 tile columns of 512 weights, so 8 ranks hold 4, 4, 4, 4, 3, 3, 3, 3 of them (the same
split for the rows of gate / up and the columns of down), and 32000 vocabulary rows are 500 tile rows: 63 on the first
four ranks, 62 on the others.
"""
import os

import numpy as np

from .bundle import Writer, ROPE_ROWS

PAIRED = ("Q4_K", "IQ4_XS")
SIDE_BYTES = {"Q4_K": 16, "Q5_K": 16, "Q6_K": 18, "IQ4_XS": 8}

MISTRAL_7B = dict(n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, inter=14336, vocab=32000,
                  eps=1e-5, theta=1e6)
PHI3_MINI = dict(n_layers=32, hidden=3072, n_heads=32, n_kv_heads=32, head_dim=96, inter=8192, vocab=32064,
                 eps=1e-5, theta=1e4)


def synth_codes(ty, n, k, rng):
    if ty == "Q4_K":
        q = np.clip(np.rint(rng.laplace(8.0, 1.5, (n, k))), 0, 15)
    elif ty == "IQ4_XS":
        q = np.clip(np.rint(rng.laplace(7.5, 1.5, (n, k))), 0, 15)
    elif ty == "Q5_K":
        q = np.clip(np.rint(rng.normal(16.0, 2.5, (n, k))), 0, 31)
    elif ty == "Q6_K":
        q = np.clip(np.rint(rng.normal(32.0, 5.0, (n, k))), 0, 63)
    else:
        raise ValueError(ty)
    return q.astype(np.uint8)


def synth_side(ty, n, k, rng):
    nb = n * k // 256
    side = rng.integers(0, 256, (nb, SIDE_BYTES[ty]), dtype=np.uint8)
    d = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if ty in ("Q4_K", "Q5_K"):
        side[:, 0:2] = d
        side[:, 2:4] = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    elif ty == "Q6_K":
        side[:, 0:16] = rng.integers(-64, 64, (nb, 16)).astype(np.int8).view(np.uint8)
        side[:, 16:18] = d
    else:
        side[:, 0:2] = d
    return side.reshape(n, -1)


def tile_split(total, unit, world, rank):
    """[lo, hi) of rank's share of `total` (a multiple of `unit`): units dealt as evenly as they go, the first
    `units % world` ranks get one more.  The runtime applies the same rule to the vocabulary (unit 64 rows)."""
    units = total // unit
    base, rem = divmod(units, world)
    start = rank * base + min(rank, rem)
    return start * unit, (start + base + (1 if rank < rem else 0)) * unit


def _shard_rows(a, lo, hi):
    return np.ascontiguousarray(a[lo:hi])


def _shard_cols(q, side, lo, hi):
    """columns lo..hi of codes [N, K] and of their side bytes (whole 256-weight super-blocks)"""
    sb = side.shape[1] // (q.shape[1] // 256)
    return np.ascontiguousarray(q[:, lo:hi]), np.ascontiguousarray(side[:, lo // 256 * sb:hi // 256 * sb])


def write_model(path, shape, fmt_attn="Q4_K", fmt_ffn=None, seed=0, tp=(0, 1), reuse_layers=False, return_weights=False):
    """Writes the bundle; returns {name: (fmt, codes, side)} of this shard's matrices if return_weights."""
    fmt_ffn = fmt_ffn or fmt_attn
    rank, world = tp
    L, D, H, Hk, Dh = shape["n_layers"], shape["hidden"], shape["n_heads"], shape["n_kv_heads"], shape["head_dim"]
    I, V = shape["inter"], shape["vocab"]
    tile_k = lambda f: 512 if f in PAIRED else 256
    assert H % world == 0 and Hk % world == 0 and I % tile_k(fmt_ffn) == 0 and V % 64 == 0
    Hl, Hkl = H // world, Hk // world
    i_lo, i_hi = tile_split(I, tile_k(fmt_ffn), world, rank)      # rows of gate / up, columns of down
    v_lo, v_hi = tile_split(V, 64, world, rank)                   # rows of lm_head
    Il, Vl = i_hi - i_lo, v_hi - v_lo
    assert Il > 0 and Vl > 0, "more ranks than tiles"
    assert (Hl * Dh) % tile_k(fmt_attn) == 0 and D % 512 == 0
    assert (Hl * Dh) % 64 == 0 and (Hkl * Dh) % 64 == 0
    w = Writer(path)
    cfg = dict(n_layers=L, hidden=D, n_heads=Hl, n_kv_heads=Hkl, head_dim=Dh, inter=Il, vocab=Vl, eps=shape["eps"],
               rope_rows=ROPE_ROWS, rope_half=Dh // 2, attn_scale=Dh ** -0.5, enc="kq_huf", tied=0, eos="2",
               tp_world=world, tp_rank=rank, vocab_full=V)
    for k, v in cfg.items():
        w.cfg(k, v)
    rng = np.random.default_rng(seed)
    emb = (rng.standard_normal((V, D)) * 0.05).astype(np.float16)
    w.add("embed", "f16", V, D, 1.0, 0, emb.tobytes())
    inv = 1.0 / (shape["theta"] ** (np.arange(0, Dh, 2, dtype=np.float64) / Dh))
    ang = np.arange(ROPE_ROWS, dtype=np.float64)[:, None] * inv[None]
    w.add("cos", "f32", ROPE_ROWS, Dh // 2, 1.0, 0, np.cos(ang).astype(np.float32).tobytes())
    w.add("sin", "f32", ROPE_ROWS, Dh // 2, 1.0, 0, np.sin(ang).astype(np.float32).tobytes())
    norms = {}
    for i in range(L):
        for nm in ("ln1", "ln2"):
            norms["l%d.%s" % (i, nm)] = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    norms["lnf"] = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    for nm, v in norms.items():
        w.add(nm, "f32", 1, D, 1.0, 0, v.tobytes())

    kept = {}
    shared = {}

    def matrix(name, fmt, n, k, mseed, rows=None, cols=None, alias=None):
        """full [n, k] matrix of seed mseed, sliced to this rank; alias: reuse the bytes already written under it"""
        if alias is not None and alias in shared:
            for suffix in ("", ".kqs"):
                enc, nn, kk, off, nb = shared[alias + suffix]
                w.lines.append("t %s%s %s %d %d %.9g %d %d %d" % (name, suffix, enc, nn, kk, 1.0, 0, off, nb))
            if return_weights:
                kept[name] = kept[alias]
            return
        r = np.random.default_rng(mseed)
        q, side = synth_codes(fmt, n, k, r), synth_side(fmt, n, k, r)
        if rows is not None:
            q, side = _shard_rows(q, *rows), _shard_rows(side, *rows)
        if cols is not None:
            q, side = _shard_cols(q, side, *cols)
        before = len(w.lines)
        w.add_kquant(name, fmt, q, side)
        for line in w.lines[before:]:
            p = line.split()
            shared[p[1]] = (p[2], int(p[3]), int(p[4]), int(p[7]), int(p[8]))
        if return_weights:
            kept[name] = (fmt, q, side)

    def qkv_rows():
        # this rank's q heads, then its k heads, then its v heads, out of the full [q | k | v] row layout
        q0 = np.arange(rank * Hl * Dh, (rank + 1) * Hl * Dh)
        k0 = H * Dh + np.arange(rank * Hkl * Dh, (rank + 1) * Hkl * Dh)
        v0 = (H + Hk) * Dh + np.arange(rank * Hkl * Dh, (rank + 1) * Hkl * Dh)
        return np.concatenate([q0, k0, v0])

    for i in range(L):
        src = 0 if reuse_layers else i
        al = (lambda s: "l0." + s) if (reuse_layers and i > 0) else (lambda s: None)
        base = seed * 100003 + src * 16
        name = "l%d.qkv" % i
        if al("qkv") and al("qkv") in shared:
            matrix(name, fmt_attn, 0, 0, 0, alias=al("qkv"))
        else:
            r = np.random.default_rng(base + 1)
            n_full = (H + 2 * Hk) * Dh
            q, side = synth_codes(fmt_attn, n_full, D, r), synth_side(fmt_attn, n_full, D, r)
            idx = qkv_rows()
            q, side = np.ascontiguousarray(q[idx]), np.ascontiguousarray(side[idx])
            before = len(w.lines)
            w.add_kquant(name, fmt_attn, q, side)
            for line in w.lines[before:]:
                p = line.split()
                shared[p[1]] = (p[2], int(p[3]), int(p[4]), int(p[7]), int(p[8]))
            if return_weights:
                kept[name] = (fmt_attn, q, side)
        matrix("l%d.o" % i, fmt_attn, D, H * Dh, base + 2, cols=(rank * Hl * Dh, (rank + 1) * Hl * Dh), alias=al("o"))
        matrix("l%d.gate" % i, fmt_ffn, I, D, base + 3, rows=(i_lo, i_hi), alias=al("gate"))
        matrix("l%d.up" % i, fmt_ffn, I, D, base + 4, rows=(i_lo, i_hi), alias=al("up"))
        matrix("l%d.down" % i, fmt_ffn, D, I, base + 5, cols=(i_lo, i_hi), alias=al("down"))
    matrix("lm_head", fmt_attn, V, D, seed * 100003 + 7777, rows=(v_lo, v_hi))
    w.close()
    if return_weights:
        kept["__embed__"] = emb
        kept["__norms__"] = norms
        kept["__rope__"] = (np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32))
    return kept if return_weights else None
