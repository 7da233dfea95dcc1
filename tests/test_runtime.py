"""The decoder runtime around the coded matrices (rt_forward and friends) against a float64 NumPy model built from
the oracle's dequantised weights: same architecture as the reference runtime's token step (RMSNorm with folded
residual, rotate-half RoPE, fp16 KV cache, grouped-query causal attention, SwiGLU)."""
import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu

SHAPE = dict(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, inter=1024, vocab=512, eps=1e-5, theta=1e4)


def ref_forward(W, ids, shape, hk_round=True):
    """All-positions logits [n, V] in float64; k and v rounded to fp16 as the cache stores them."""
    L, D, H, Hk, Dh, I = (shape[k] for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "inter"))
    emb, norms, (cos, sin) = W["__embed__"], W["__norms__"], W["__rope__"]
    # a matrix is (format, codes, side bytes), or float weights that some other path has already dequantised
    deq = lambda name: (W[name] if isinstance(W[name], np.ndarray)
                        else orc.dequant(W[name][0], W[name][1], W[name][2])).astype(np.float64)
    h = emb[ids].astype(np.float64)
    n = len(ids)

    def rms(x, g):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + shape["eps"]) * g

    def rope(x, p):   # x [heads, Dh]
        half = Dh // 2
        a, b = x[:, :half], x[:, half:]
        c, s = cos[p][None].astype(np.float64), sin[p][None].astype(np.float64)
        return np.concatenate([a * c - b * s, b * c + a * s], 1)

    for l in range(L):
        xn = rms(h, norms["l%d.ln1" % l])
        qkv = xn @ deq("l%d.qkv" % l).T
        q = qkv[:, :H * Dh].reshape(n, H, Dh)
        k = qkv[:, H * Dh:(H + Hk) * Dh].reshape(n, Hk, Dh)
        v = qkv[:, (H + Hk) * Dh:].reshape(n, Hk, Dh)
        q = np.stack([rope(q[p], p) for p in range(n)])
        k = np.stack([rope(k[p], p) for p in range(n)]).astype(np.float16).astype(np.float64)
        v = v.astype(np.float16).astype(np.float64)
        att = np.zeros((n, H, Dh))
        for p in range(n):
            for hd in range(H):
                kh = hd // (H // Hk)
                s = (k[:p + 1, kh] @ q[p, hd]) * Dh ** -0.5
                e = np.exp(s - s.max())
                att[p, hd] = (e / e.sum()) @ v[:p + 1, kh]
        h = h + att.reshape(n, H * Dh) @ deq("l%d.o" % l).T
        xn = rms(h, norms["l%d.ln2" % l])
        g, u = xn @ deq("l%d.gate" % l).T, xn @ deq("l%d.up" % l).T
        h = h + (g / (1 + np.exp(-g)) * u) @ deq("l%d.down" % l).T
    return rms(h, norms["lnf"]) @ deq("lm_head").T


@pytest.mark.parametrize("fmt_attn,fmt_ffn", [("Q4_K", "Q4_K"), ("Q5_K", "Q6_K")])
def test_forward_matches_numpy_model(tmp_path, fmt_attn, fmt_ffn):
    helpers.build_library()
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen
    W = modelgen.write_model(str(tmp_path / "m"), SHAPE, fmt_attn, fmt_ffn, seed=3, return_weights=True)
    ids = np.random.default_rng(1).integers(0, SHAPE["vocab"], 11).astype(np.int32)
    ref = ref_forward(W, ids, SHAPE)
    with lw.Bundle(str(tmp_path / "m"), max_ctx=64, max_batch=8) as b:
        assert b.vocab == SHAPE["vocab"] and b.pos == 0
        full = b.forward(ids, all_logits=True)                       # two passes: 8 + 3 tokens
        assert b.pos == 11 and full.shape == ref.shape
        assert helpers.rel_err(full, ref) <= 5e-3
        assert (full.argmax(1) == ref.argmax(1)).mean() >= 0.9
        b.reset()
        step = np.stack([b.forward(ids[i:i + 1]) for i in range(len(ids))])   # token by token
        # attention is per query whatever the pass carries; the matrices differ in how the activations are rounded
        # (16-bit block fixed point for one token, fp16 on the tensor cores for eight): both within the product bar
        assert helpers.rel_err(step, full) <= 1e-3
        assert b.stat("graph_captures") >= 1 and b.stat("graph_launches") >= 9   # replayed CUDA graphs, same logits
        b.set_pos(5)                                                 # rewind: the cache below 5 is kept
        assert b.pos == 5
        again = b.forward(ids[5:], all_logits=True)
        assert helpers.rel_err(again, full[5:]) <= 1e-3
        b.reset()
        with pytest.raises(IndexError):
            b.forward(np.zeros(65, np.int32))                        # context overflow: the reference's -1
        assert b.kernel_error() == 0


def test_prompt_lookup_equals_greedy(tmp_path):
    """Speculation must not change the output: drafts are only accepted where they equal the greedy choice."""
    helpers.build_library()
    import lazyweights_b200 as lw
    from lazyweights_b200 import modelgen, speculate
    modelgen.write_model(str(tmp_path / "m"), SHAPE, "IQ4_XS", "IQ4_XS", seed=5)
    rng = np.random.default_rng(3)
    motif = rng.integers(0, SHAPE["vocab"], 6)
    prompt = np.concatenate([motif, rng.integers(0, SHAPE["vocab"], 4), motif, motif[:3]]).astype(np.int32)
    with lw.Bundle(str(tmp_path / "m"), max_ctx=128, max_batch=8) as b:
        plain = speculate.greedy(b, prompt, 24)
        spec, passes, accepted = speculate.prompt_lookup(b, prompt, 24, n_draft=7, ngram=3)
        assert spec == plain
        assert passes <= 24 and accepted >= 0
        cached, passes_c, accepted_c = speculate.prompt_lookup(b, prompt, 24, n_draft=7, drafter="ngramcache")
        assert cached == plain and passes_c <= 24 and accepted_c >= 0
        # the same tokens when the runtime picks them itself, pass after pass without the host (80 tokens: the passes
        # cross a boundary of the attention's 64-position chunks, i.e. more than one captured graph)
        long_plain = speculate.greedy(b, prompt, 80)
        assert long_plain[:24] == plain
        pos = b.pos
        assert speculate.greedy(b, prompt, 80, on_device=True) == long_plain
        assert b.pos == pos
        with pytest.raises(IndexError):
            b.decode_greedy(1, 128)                                       # beyond the context: refused, nothing launched
        with pytest.raises(lw.LwError):
            b.decode_greedy(SHAPE["vocab"], 1)


def test_bundle_built_from_a_gguf_runs(tmp_path):
    """A synthetic llama-architecture GGUF (permuted q / k rows, separate q / k / v of one type, Q6_K embedding) goes
    through the bundle builder and the runtime; logits against the NumPy model on gguf-py's own dequantised tensors."""
    import os
    import sys
    helpers.build_library()
    import gguf
    import lazyweights_b200 as lw
    from lazyweights_b200 import gguf_bundle
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import synth_gguf as sg
    path = str(tmp_path / "m.gguf")
    made = sg.write(path, **sg.CASES["llama_fused"])
    gguf_bundle.build_bundle(path, str(tmp_path / "b"), check=True)
    shape = dict(n_layers=sg.LAYERS, hidden=sg.HIDDEN, n_heads=sg.HEADS, n_kv_heads=sg.KV_HEADS, head_dim=sg.HEAD_DIM,
                 inter=sg.INTER, vocab=sg.VOCAB, eps=1e-5, theta=1e6)

    def dq(name, heads=None):
        ty, rows, cols, b = made[name]
        w = gguf.quants.dequantize(b, getattr(gguf.GGMLQuantizationType, ty)).reshape(rows, cols)
        if heads:                                                     # GGUF row order -> rotate-half order
            w = w.reshape(heads, rows // heads // 2, 2, cols).swapaxes(1, 2).reshape(rows, cols)
        return w

    W = {"__embed__": dq("token_embd.weight").astype(np.float16), "__norms__": {"lnf": made["output_norm.weight"][3]}}
    for i in range(sg.LAYERS):
        p = "blk.%d." % i
        W["l%d.qkv" % i] = np.concatenate([dq(p + "attn_q.weight", sg.HEADS), dq(p + "attn_k.weight", sg.KV_HEADS),
                                           dq(p + "attn_v.weight")])
        for ours, theirs in (("o", "attn_output"), ("gate", "ffn_gate"), ("up", "ffn_up"), ("down", "ffn_down")):
            W["l%d.%s" % (i, ours)] = dq(p + theirs + ".weight")
        W["__norms__"]["l%d.ln1" % i] = made[p + "attn_norm.weight"][3]
        W["__norms__"]["l%d.ln2" % i] = made[p + "ffn_norm.weight"][3]
    W["lm_head"] = dq("output.weight")
    inv = 1.0 / (1e6 ** (np.arange(0, sg.HEAD_DIM, 2, dtype=np.float64) / sg.HEAD_DIM))
    ang = np.arange(64, dtype=np.float64)[:, None] * inv[None]
    W["__rope__"] = (np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32))
    ids = np.random.default_rng(6).integers(0, sg.VOCAB, 9).astype(np.int32)
    ref = ref_forward(W, ids, shape)
    with lw.Bundle(str(tmp_path / "b"), max_ctx=64, max_batch=8) as b:
        got = b.forward(ids, all_logits=True)
        assert helpers.rel_err(got, ref) <= 5e-3
        assert b.kernel_error() == 0
